"""ZeRO logic on CPU ranks (gloo): W in {1, 2, 4} give the same loss curve and parameters for the
same global batch, for ZeRO-3, ZeRO-2.5, gradient accumulation and the offloaded optimizer; the
launcher's watchdog tears a job down when a rank raises, exits or stalls."""
import os
import pickle
import time

import numpy as np
import pytest

from tests.dist_helpers import run_spawn, train_worker


def run(world, tmp_path, cfg, tag):
    out = tmp_path / f"{tag}_w{world}"
    out.mkdir()
    codes = run_spawn(train_worker, world, str(out), cfg)
    assert codes == [0] * world, codes
    res = [pickle.load(open(out / f"r{r}.pkl", "rb")) for r in range(world)]
    losses = np.mean([r["losses"] for r in res], axis=0)
    for r in res[1:]:
        for a, b in zip(res[0]["params"], r["params"]):
            np.testing.assert_array_equal(a, b)      # every rank gathers the same parameters
    return losses, res[0]["params"], res


@pytest.mark.parametrize("cfg,tag", [
    (dict(zero="3"), "z3"),
    (dict(zero="2.5", model=dict(zero25_replica_ratio=0.3)), "z25"),
    (dict(zero="2.5", model=dict(zero25_replica_ratio=1.0)), "z2"),
    (dict(zero="3", opt="cpu"), "offload"),
    (dict(zero="3", model=dict(tie_embeddings=False, keep_layer_num=2)), "untied"),
])
def test_world_sizes_agree(tmp_path, cfg, tag):
    base_l, base_p, _ = run(1, tmp_path, cfg, tag)
    for world in (2, 4):
        l, p, res = run(world, tmp_path, cfg, tag)
        np.testing.assert_allclose(l, base_l, rtol=2e-5, atol=2e-6)
        for a, b in zip(p, base_p):
            np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-6)
        if cfg.get("zero") == "3":
            assert res[0]["gathered"] > 0 and res[0]["reduced"] > 0


def test_keep_params_until_backward_gathers_each_block_once(tmp_path):
    """keep_params_until_backward: same losses and parameters bit for bit, fewer bytes gathered (also with
    two micro-batches per step, where every forward / backward pair gathers once)."""
    for accum in (1, 2):
        l0, p0, r0 = run(2, tmp_path, dict(zero="3", accum=accum), f"regather{accum}")
        l1, p1, r1 = run(2, tmp_path, dict(zero="3", accum=accum, model=dict(keep_params_until_backward=True)),
                         f"keep{accum}")
        np.testing.assert_array_equal(l0, l1)
        for a, b in zip(p0, p1):
            np.testing.assert_array_equal(a, b)
        assert r1[0]["gathered"] < 0.75 * r0[0]["gathered"]


def test_accumulation_across_ranks(tmp_path):
    base_l, base_p, _ = run(1, tmp_path, dict(zero="3"), "acc_ref")
    l, p, _ = run(2, tmp_path, dict(zero="3", accum=2), "acc")
    np.testing.assert_allclose(l, base_l, rtol=2e-5, atol=2e-6)
    for a, b in zip(p, base_p):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-6)


def test_checkpoint_written_by_two_ranks_reshards_to_one(tmp_path):
    from create_llm_by_cupy_b200.utils import checkpoint as ckpt

    d = tmp_path / "ck2"
    _, p2, _ = run(2, tmp_path, dict(zero="3", save_dir=str(d)), "save")
    assert (d / "model_shard_rank1.pkl.gz").exists() and (d / "optimizer_rank1.pkl.gz").exists()
    full = ckpt.shards_to_param_list(str(d))
    for a, b in zip(full, p2):
        np.testing.assert_array_equal(a.numpy(), b)
    d1 = tmp_path / "ck1"
    ckpt.reshard_checkpoint(str(d), str(d1), 1)
    for a, b in zip(ckpt.shards_to_param_list(str(d1)), p2):
        np.testing.assert_array_equal(a.numpy(), b)


@pytest.mark.parametrize("kind", ["raise", "exit", "stall"])
def test_launcher_watchdog_detects_failed_rank(tmp_path, kind):
    from create_llm_by_cupy_b200.parallel.trainer import TrainMultiGPU, WorkerFailure
    from tests.dist_helpers import TINY

    launcher = TrainMultiGPU(TINY, use_devices=[0, 1], batch_size=2, accum_step=1, backend="gloo", console=False,
                             fault=dict(rank=1, iter=1, kind=kind, seconds=600), heartbeat_timeout_s=6.0,
                             collective_timeout_s=30.0, heartbeat_dir=str(tmp_path), synthetic_samples=32,
                             master_port=23000 + os.getpid() % 5000 + {"raise": 0, "exit": 1, "stall": 2}[kind])
    t0 = time.time()
    with pytest.raises(WorkerFailure):
        launcher.fit(2 * 2 * 6)
    assert time.time() - t0 < 90


def test_launcher_runs_clean_job(tmp_path):
    from create_llm_by_cupy_b200.parallel.trainer import TrainMultiGPU
    from tests.dist_helpers import TINY

    launcher = TrainMultiGPU(TINY, use_devices=[0, 1], batch_size=2, accum_step=2, backend="gloo", console=False,
                             vali=True, vali_step=2, save=True, save_step=3, save_dir=str(tmp_path / "ck"),
                             result_dir=str(tmp_path), synthetic_samples=64, master_port=28000 + os.getpid() % 1000,
                             metrics_path=str(tmp_path / "metrics.jsonl"))
    codes = launcher.fit(2 * 2 * 2 * 4)
    assert codes == [0, 0]
    assert (tmp_path / "ck" / "model_shard_rank1.pkl.gz").exists()
    lines = open(tmp_path / "metrics.jsonl").read().strip().splitlines()
    assert any("validation" in ln for ln in lines) and any("tokens_per_s" in ln for ln in lines)
    # the generation split is used: every validation point decodes from a prompt of that split
    from create_llm_by_cupy_b200.utils import checkpoint as ckpt
    res = ckpt.read_pickle_gzip(str(tmp_path / "result_rank0.pkl.gz"))
    assert len(res["losses"]) == 4 and res["iteration"] == 4
    assert len(res["generation"]) == 2 and all(len(g["tokens"]) > 0 for g in res["generation"])
    assert any("generated_tokens" in ln for ln in lines)


def test_launcher_resumes_at_the_saved_iteration_and_data_position(tmp_path):
    """A job stopped after 3 of 6 iterations and resumed produces the losses of the uninterrupted job."""
    from create_llm_by_cupy_b200.parallel.trainer import TrainMultiGPU
    from create_llm_by_cupy_b200.utils import checkpoint as ckpt
    from tests.dist_helpers import TINY

    common = dict(use_devices=[0], batch_size=2, accum_step=1, backend="gloo", console=False, synthetic_samples=32,
                  warm_up=2)
    whole = tmp_path / "whole"
    TrainMultiGPU(TINY, result_dir=str(whole), **common).fit(2 * 6)
    ref = ckpt.read_pickle_gzip(str(whole / "result_rank0.pkl.gz"))["losses"]
    assert len(ref) == 6
    ck = tmp_path / "ck"
    first = tmp_path / "first"
    a = TrainMultiGPU(TINY, result_dir=str(first), save=True, save_step=3, save_dir=str(ck), **common)
    a.args["stop_after"] = 3
    a.fit(2 * 6)
    second = tmp_path / "second"
    TrainMultiGPU(TINY, result_dir=str(second), resume_dir=str(ck), **common).fit(2 * 6)
    got = ckpt.read_pickle_gzip(str(second / "result_rank0.pkl.gz"))
    assert got["iteration"] == 6
    np.testing.assert_allclose(got["losses"], ref[3:], rtol=1e-5, atol=1e-6)
