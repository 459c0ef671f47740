"""Trainer on CPU: single-process steps against the NumPy oracle's AdamW, gradient accumulation,
NaN skip, ZeRO-2.5 equivalence, checkpoint round trip and resharding."""
import math
import os

import numpy as np
import pytest
import torch

from create_llm_by_cupy_b200.models.oracle_np import Oracle, OracleConfig, cosine_lr
from create_llm_by_cupy_b200.parallel.trainer import Trainer
from create_llm_by_cupy_b200.utils import checkpoint as ckpt
from create_llm_by_cupy_b200.utils.data import padding_proceccing, synthetic_token_stream

TINY = dict(vocab_size=64, hidden_size=32, layer_num=2, time_size=16, q_head=4, kv_head=2, padding_id=2,
            dropout_rate=0, half_float=False, dtype="fp32", ffn_size=48, tie_embeddings=False, seed=3,
            ce_chunk_size=24)
HP = dict(lr_max=3e-3, lr_mini=3e-4, weight_decay=0.1, warm_up=3, total_steps=10, beta1=0.9, beta2=0.95,
          epsilon=1e-6, max_grads=1.0)


def batches(n, B=4, seed_split="train"):
    ids = synthetic_token_stream(n * B, TINY["time_size"], TINY["vocab_size"], seed_split, TINY["padding_id"], low=3)
    out = []
    for i in range(n):
        chunk = ids[i * B:(i + 1) * B]
        out.append(padding_proceccing(chunk, np.full(B, TINY["time_size"]), TINY["padding_id"]))
    return out


def full_params(trainer):
    trainer.manager.materialize_all()
    ps = [p.detach().double().numpy().copy() for p in trainer.model.params]
    trainer.manager.release_all()
    return ps


def test_ten_adam_steps_match_oracle():
    tr = Trainer(TINY, device="cpu", **HP)
    orc = Oracle(OracleConfig.from_model_dic(TINY), full_params(tr))
    orc.init_adam()
    bs = batches(10)
    for step, (x, t, pa) in enumerate(bs, 1):
        out = tr.train_step([(x, t, pa)])
        ref_loss = orc.forward(x.numpy(), t.numpy(), pa.numpy())
        g = orc.backward()
        orc.adam_step(g, cosine_lr(step, HP["lr_max"], HP["lr_mini"], HP["warm_up"], HP["total_steps"]),
                      HP["beta1"], HP["beta2"], HP["epsilon"], HP["weight_decay"], HP["max_grads"])
        assert abs(out["loss"] - ref_loss) < 2e-4 * max(1.0, abs(ref_loss)), (step, out["loss"], ref_loss)
        assert not out["skipped"]
    for a, b in zip(full_params(tr), orc.p):
        np.testing.assert_allclose(a, b, rtol=2e-3, atol=2e-5)


def test_grad_accumulation_equals_big_batch_of_same_tokens():
    bs = batches(2)
    tr1 = Trainer(TINY, device="cpu", accum_step=2, **HP)
    o1 = tr1.train_step(bs)
    tr2 = Trainer(TINY, device="cpu", accum_step=1, **HP)
    big = tuple(torch.cat([bs[0][i], bs[1][i]]) for i in range(3))
    o2 = tr2.train_step([big])
    assert abs(o1["loss"] - o2["loss"]) < 1e-5
    for a, b in zip(full_params(tr1), full_params(tr2)):
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)


def test_nan_step_is_skipped_and_loss_scale_shrinks():
    tr = Trainer(TINY, device="cpu", GradScale_dic=dict(StartScale=10, enabled=True), **HP)
    before = full_params(tr)
    tr.inject_nan_next = True
    out = tr.train_step(batches(1))
    assert out["skipped"] and tr.scaler.Scale == pytest.approx(7.0) and tr.optimizer.t == 0
    for a, b in zip(before, full_params(tr)):
        np.testing.assert_array_equal(a, b)
    out = tr.train_step(batches(1))
    assert not out["skipped"] and tr.optimizer.t == 1


@pytest.mark.parametrize("ratio,policy", [(0.3, "largest_first"), (1.0, "first"), (0.5, "embedding_first")])
def test_zero25_single_rank_matches_zero3(ratio, policy):
    bs = batches(3)
    ref = Trainer(TINY, device="cpu", accum_step=1, **HP)
    md = dict(TINY, zero25_replica_ratio=ratio, zero25_replica_policy=policy)
    z25 = Trainer(md, device="cpu", zero_stage="2.5", **HP)
    assert z25.manager.replicated_param_indices
    for b in bs:
        a, c = ref.train_step([b]), z25.train_step([b])
        assert abs(a["loss"] - c["loss"]) < 1e-5
    for a, b in zip(full_params(ref), full_params(z25)):
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)


def test_checkpoint_roundtrip_resume_flat_and_reshard(tmp_path):
    bs = batches(4)
    tr = Trainer(TINY, device="cpu", **HP)
    tr.train_step([bs[0]])
    tr.train_step([bs[1]])
    d = str(tmp_path / "ck")
    tr.save(d)
    for f in ("model_shard_rank0.pkl.gz", "optimizer_rank0.pkl.gz", "trainer_state.pkl.gz"):
        assert os.path.exists(os.path.join(d, f))
    shard = ckpt.read_pickle_gzip(ckpt.model_shard_path(d, 0))
    for k in ("param_shard_f16", "rank", "world_size", "shard_size", "padded_total", "param_offsets",
              "param_shapes", "param_sizes"):
        assert k in shard
    opt = ckpt.read_pickle_gzip(ckpt.optimizer_path(d, 0))
    assert set(("m", "v", "w_fp32", "t")) <= set(opt)
    # resume: a fresh trainer continues exactly like the original
    tr2 = Trainer(dict(TINY, seed=77), device="cpu", **HP)
    st = tr2.load(d)
    assert st["iteration"] == 2 and tr2.optimizer.t == 2
    a, b = tr.train_step([bs[2]]), tr2.train_step([bs[2]])
    assert abs(a["loss"] - b["loss"]) < 1e-6
    for x, y in zip(full_params(tr), full_params(tr2)):
        np.testing.assert_allclose(x, y, rtol=1e-6, atol=1e-7)
    # shards -> flat (the reference's resume format) -> model
    flat = str(tmp_path / "flat_params_f16.pkl.gz")
    ckpt.shards_to_flat(d, flat)
    from create_llm_by_cupy_b200.models.model import Cupa_ver4
    m = Cupa_ver4(TINY, param_path=flat, device="cpu")
    saved = ckpt.shards_to_param_list(d)
    for p, q in zip(m.params, saved):
        np.testing.assert_allclose(p.numpy(), q.numpy(), rtol=2e-3, atol=2e-3)
    # reshard 1 -> 4 -> 1 keeps parameters and optimizer state
    d4, d1 = str(tmp_path / "w4"), str(tmp_path / "w1")
    ckpt.reshard_checkpoint(d, d4, 4)
    assert os.path.exists(ckpt.optimizer_path(d4, 3))
    ckpt.reshard_checkpoint(d4, d1, 1)
    for p, q in zip(ckpt.shards_to_param_list(d1), saved):
        np.testing.assert_array_equal(p.numpy(), q.numpy())
    o1 = ckpt.read_pickle_gzip(ckpt.optimizer_path(d1, 0))
    np.testing.assert_array_equal(o1["m"], opt["m"])
    # flat -> shards for 2 ranks
    d2 = str(tmp_path / "w2")
    ckpt.flat_to_shards(flat, d2, [tuple(p.shape) for p in m.params], m.unit_defs(), 2, dtype_name="fp32")
    for p, q in zip(ckpt.shards_to_param_list(d2), saved):
        np.testing.assert_allclose(p.numpy(), q.numpy(), rtol=2e-3, atol=2e-3)


def test_weights_without_optimizer_file_reseed_the_master_copy(tmp_path):
    """flat -> shards writes no optimizer file. Loading it must make the fp32 master follow the loaded
    weights: the first AdamW step then moves the parameters by about one learning-rate step instead of
    replacing them with values derived from the randomly initialised master."""
    src = Trainer(TINY, device="cpu", **HP)
    for b in batches(3):
        src.train_step([b])
    flat = str(tmp_path / "flat.pkl.gz")
    src.manager.materialize_all()
    src.model.save_weights_to_flat_file(flat)
    shapes = [tuple(p.shape) for p in src.model.params]
    src.manager.release_all()
    d = str(tmp_path / "shards")
    ckpt.flat_to_shards(flat, d, shapes, src.model.unit_defs(), 1, dtype_name="fp32")
    assert not os.path.exists(ckpt.optimizer_path(d, 0))
    tr = Trainer(dict(TINY, seed=123), device="cpu", **HP)
    tr.load(d)
    loaded = full_params(tr)
    np.testing.assert_array_equal(tr.optimizer.master_weight_shard.numpy(), tr.manager.param_shard_f16.float().numpy())
    assert tr.optimizer.t == 0 and float(tr.optimizer.m.abs().max()) == 0.0
    tr.train_step([batches(1)[0]])
    for a, b in zip(full_params(tr), loaded):
        assert np.abs(a - b).max() <= 3 * HP["lr_max"] * (1 + np.abs(b).max())


def test_resume_restores_rng_states_and_iteration(tmp_path):
    tr = Trainer(TINY, device="cpu", **HP)
    tr.train_step([batches(1)[0]])
    d = str(tmp_path / "ck")
    torch.manual_seed(1234)
    np.random.seed(99)
    tr.save(d)
    want_t, want_n = torch.rand(3), np.random.rand(3)
    torch.manual_seed(1)
    np.random.seed(1)
    tr2 = Trainer(dict(TINY, seed=5), device="cpu", **HP)
    tr2.load(d)
    assert tr2.iteration == 1
    assert torch.equal(torch.rand(3), want_t)
    np.testing.assert_array_equal(np.random.rand(3), want_n)


def test_replica_selection_stops_once_the_target_is_reached():
    """Same rule as the reference (model/ZeRO2_5.py:863-892): take parameters in the policy's order until
    the running total has reached int(total * ratio); the last one may overshoot, at least one is taken."""
    from create_llm_by_cupy_b200.parallel.layout import select_replicated_params

    sizes = [50, 10, 30, 5, 40, 15]          # total 150

    def restated(order, ratio):
        target, acc, out = int(sum(sizes) * ratio), 0, []
        for i in order:
            if acc >= target:
                break
            out.append(i)
            acc += sizes[i]
        return sorted(out)

    by_size = sorted(range(6), key=lambda i: (-sizes[i], i))
    for ratio in (0.01, 0.3, 0.34, 0.5, 0.9):
        assert select_replicated_params(sizes, [2], ratio, "largest_first") == restated(by_size, ratio)
        assert select_replicated_params(sizes, [2], ratio, "first") == restated(list(range(6)), ratio)
        assert select_replicated_params(sizes, [2], ratio, "last") == restated(list(range(5, -1, -1)), ratio)
        emb_first = [2] + [i for i in by_size if i != 2]
        assert select_replicated_params(sizes, [2], ratio, "embedding_first") == restated(emb_first, ratio)
    # a ratio below the embedding's share still replicates the embedding (never silently plain ZeRO-3)
    assert select_replicated_params(sizes, [2], 0.05, "embedding_first") == [2]
    assert select_replicated_params(sizes, [2], 0.0, "first") == []
    assert select_replicated_params(sizes, [2], 1.0, "last") == list(range(6))


def test_validation_and_generation_through_trainer():
    tr = Trainer(TINY, device="cpu", **HP)
    v = tr.validate(batches(2, seed_split="validation"))
    assert math.isfinite(v) and abs(v - math.log(TINY["vocab_size"])) < 1.0
    out = tr.generate([5, 6, 7], greedy=True, max_new_tokens=5)
    assert len(out) == 5


def test_gradient_buffer_pool_rotates_two_buffers_deterministically():
    """With rotate=2 a buffer handed back is not the next one handed out (its collective may still be
    reading it), and the sequence of allocations depends on the call sequence only."""
    from create_llm_by_cupy_b200.parallel.zero import _Pool
    made = []

    def alloc(n, dtype):
        made.append(n)
        return torch.zeros(n, dtype=dtype)

    pool = _Pool(torch.float32, "cpu", alloc, rotate=2)
    a = pool.get(16)
    pool.put(a)
    b = pool.get(16)              # second buffer although the first is free again
    assert b.t.data_ptr() != a.t.data_ptr() and made == [16, 16]
    pool.put(b)
    c = pool.get(16)              # first in, first out
    assert c.t.data_ptr() == a.t.data_ptr()
    pool.put(c)
    d = pool.get(16)
    assert d.t.data_ptr() == b.t.data_ptr() and made == [16, 16]
    single = _Pool(torch.float32, "cpu", alloc, rotate=1)
    x = single.get(8)
    single.put(x)
    assert single.get(8).t.data_ptr() == x.t.data_ptr()


def test_gradient_bucket_limit_splits_a_unit_into_parts_that_cover_it_once():
    tr = Trainer(dict(TINY, grad_bucket_elems=1000), device="cpu", **HP)
    mgr = tr.manager
    assert mgr._split_range(0, 2504) == [(0, 1000), (1000, 2000), (2000, 2504)]
    assert mgr._split_range(8, 8) == [] and mgr._split_range(16, 400) == [(16, 400)]

    class B:
        flushed = [(1200, 2400), (4000, 4800)]
    parts = mgr._unflushed_parts(B, 5600)
    covered = sorted(parts + B.flushed)
    assert covered[0][0] == 0 and covered[-1][1] == 5600
    assert all(a[1] == b[0] for a, b in zip(covered[:-1], covered[1:]))          # no gap, no overlap
    assert all(hi - lo <= 1000 for lo, hi in parts)
    # inside a block's unit the MLP weights are one contiguous tail (what the early flush reduces)
    lay = mgr.layout
    uid = mgr.uid_of_name["block0"]
    feed = tr.model.block_modules(0)[1]
    offs = sorted((lay.slots[i].offset, lay.slots[i].offset + lay.slots[i].size) for i in feed._zero3_param_indices)
    others = [lay.slots[i] for i in lay.units[uid].param_indices if i not in feed._zero3_param_indices]
    assert all(s.offset + s.size <= offs[0][0] for s in others)


def test_forward_unit_order_and_ranges_cover_the_shard():
    from create_llm_by_cupy_b200.parallel.trainer import Trainer
    md = dict(vocab_size=64, hidden_size=32, layer_num=3, time_size=16, q_head=4, kv_head=2, ffn_size=64,
              padding_id=0, dropout_rate=0, tie_embeddings=True, seed=0)
    tr = Trainer(md, device="cpu")
    mgr = tr.manager
    order = mgr.forward_unit_order()
    names = [mgr.unit_names[u] for u in order]
    assert names[0] == "embedding"
    blocks = [n for n in names if n.startswith("block")]
    assert blocks == sorted(blocks, key=lambda n: int("".join(c for c in n if c.isdigit())))
    assert names.index(blocks[-1]) < names.index(next(n for n in names if n.startswith("final_norm")))
    ranges = sorted(mgr.layout.unit_shard_range(u) for u in order)
    assert ranges[0][0] == 0 and ranges[-1][1] == mgr.shard_size
    assert all(a[1] == b[0] for a, b in zip(ranges[:-1], ranges[1:]))


def test_fused_gather_region_is_the_chunks_that_hold_the_weight():
    """Host arithmetic of the all-gather fused into a GEMM: the kernel copies whole 32 KiB chunks of
    the per-rank slices, starting with the one that holds the first byte of the weight."""
    import ctypes
    from create_llm_by_cupy_b200.ops import native
    try:
        lib = native.lib()
    except OSError:
        pytest.skip("native library not loadable here")
    out = (ctypes.c_ulonglong * 3)()
    chunk = 32 * 1024
    slice_bytes = 5 * chunk + 4096            # the last chunk of every slice is short
    W = 4
    # weight inside slice 1, from the middle of its chunk 1 to the middle of its chunk 3
    b_off = slice_bytes + chunk + 100 * 16
    b_bytes = 2 * chunk
    assert lib.b200_ag_region(ctypes.c_ulonglong(slice_bytes), W, ctypes.c_ulonglong(b_off), ctypes.c_ulonglong(b_bytes), out) == 0
    assert (out[0], out[1], out[2]) == (slice_bytes + chunk, slice_bytes + 4 * chunk, 3)
    # weight that runs over the short tail of slice 0 into slice 1
    b_off = 4 * chunk + 16
    b_bytes = 2 * chunk
    lib.b200_ag_region(ctypes.c_ulonglong(slice_bytes), W, ctypes.c_ulonglong(b_off), ctypes.c_ulonglong(b_bytes), out)
    assert out[0] == 4 * chunk and out[1] == slice_bytes + chunk and out[2] == 3     # chunks (0,4), (0,5 short), (1,0)


def test_copy_form_reduce_scatter_takes_a_bucket_whole_and_every_rank_takes_the_same_branch():
    """The copy-engine form of the reduce-scatter is not cut by ``grad_bucket_elems`` (a range covers only some
    ranks' slices and every part costs two cross-GPU barriers) unless parts are flushed early; and the choice
    between the copy and the pull form depends only on numbers every rank computes alike."""
    from create_llm_by_cupy_b200.parallel import symm as S

    tr = Trainer(dict(TINY, grad_bucket_elems=1000), device="cpu", **HP)
    mgr = tr.manager

    class Fake:
        reduce_mode = "copy"
    mgr.fused = Fake()
    try:
        assert mgr._split_range(0, 2504) == [(0, 2504)]
        mgr.early_bucket_flush = True
        assert mgr._split_range(0, 2504) == [(0, 1000), (1000, 2000), (2000, 2504)]
        mgr.early_bucket_flush = False
        Fake.reduce_mode = "pull"
        assert mgr._split_range(0, 2504) == [(0, 1000), (1000, 2000), (2000, 2504)]
    finally:
        mgr.fused = None

    # branch selection and the share arithmetic of FusedCollectives.reduce_scatter_accumulate, launches stubbed out
    calls = []

    class Lib:
        def b200_symm_reduce_scatter_staged(self, *a):
            calls.append(("copy", a[5].value, a[6].value, a[15].value))      # lo, hi, part
            return 0

        def b200_symm_reduce_scatter_range(self, *a):
            calls.append(("pull", a[6].value, a[7].value))
            return 0

    class T:      # the few tensor attributes the method reads
        def __init__(self, n, dtype=torch.bfloat16):
            self._n, self.dtype = n, dtype

        def numel(self):
            return self._n

        def data_ptr(self):
            return 256

    class Heap:
        table = None

        def offset_of(self, t):
            return 0

    picks = []
    for rank in (0, 1, 2, 3):
        fc = S.FusedCollectives.__new__(S.FusedCollectives)
        fc.lib, fc.world_size, fc.rank, fc.wait_ns, fc.launches, fc.copies = Lib(), 4, rank, 1, 0, 0
        fc.reduce_mode, fc.copy_min_bytes, fc.rs_epoch, fc.stage_epoch, fc.rs_blocks, fc.rs_local_blocks = "copy", 1024, 0, 0, 4, 8
        fc._heap, fc._stage, fc.device = Heap(), None, torch.device("cpu")
        fc.reserve_stage = lambda part, fc=fc: T(part * 3)
        real_bump, real_check, real_stream = S.native.bump, S.native.check, S.native.stream_ptr
        S.native.bump = lambda *a, **k: None
        S.native.check = lambda rc, what: None
        S.native.stream_ptr = lambda: None
        try:
            calls.clear()
            fc.reduce_scatter_accumulate(T(1000), T(4000), False)                              # 2000 B per share: copy
            fc.reduce_scatter_accumulate(T(1000), T(4000), False, elem_range=(0, 1200))       # largest share 1000: copy
            fc.reduce_scatter_accumulate(T(1000), T(4000), False, elem_range=(992, 1200))     # largest share 200: pull
        finally:
            S.native.bump, S.native.check, S.native.stream_ptr = real_bump, real_check, real_stream
        picks.append([c[0] for c in calls])
        assert calls[0] == ("copy", 0, 4000, 1000) and calls[1] == ("copy", 0, 1200, 1000) and calls[2][0] == "pull"
    assert all(p == picks[0] for p in picks)          # every rank takes the same branch for the same call
