"""Fused peer-memory collectives. On one GPU the W ranks are virtual: W heaps on the same device
and ONE launch whose gridDim.y enumerates the ranks. On >= 2 GPUs the real thing runs in child
processes (NCCL for the baseline comparison, NVLS off)."""
import os
import subprocess
import sys

import pytest
import torch

from create_llm_by_cupy_b200.ops import native

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("W", [2, 4, 8])
def test_virtual_ranks_reduce_scatter_store_accumulate_and_stats(W):
    from create_llm_by_cupy_b200.parallel.symm import LocalVirtualRanks

    vr = LocalVirtualRanks(W)
    n_slice = 8 * 1000 + 8
    off, buckets = vr.alloc(n_slice * W, torch.bfloat16)
    for r, b in enumerate(buckets):
        b.copy_((torch.randn(n_slice * W, generator=torch.Generator().manual_seed(r)) * 2).to(torch.bfloat16))
    full = torch.stack([b.float() for b in buckets]).sum(0)
    # store (bf16) with statistics
    dsts = [torch.empty(n_slice, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    stats = [torch.zeros(2, device="cuda") for _ in range(W)]
    vr.reduce_scatter(off, n_slice, dsts, stats=stats, do_stats=True)
    torch.cuda.synchronize()
    assert native.read_status() == (0, 0)
    for r in range(W):
        ref = full[r * n_slice:(r + 1) * n_slice]
        assert (dsts[r].float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
        assert abs(stats[r][0].item() - (dsts[r].float() ** 2).sum().item()) <= 1e-3 * stats[r][0].item()
        assert stats[r][1].item() == 0
    # accumulate into fp32 twice
    acc = [torch.ones(n_slice, device="cuda") for _ in range(W)]
    vr.reduce_scatter(off, n_slice, acc, accumulate=True)
    vr.reduce_scatter(off, n_slice, acc, accumulate=True, stats=stats, do_stats=False)
    torch.cuda.synchronize()
    for r in range(W):
        ref = 1 + 2 * full[r * n_slice:(r + 1) * n_slice]
        assert (acc[r] - ref).abs().max().item() < 1e-3
    # a NaN in one rank's bucket is flagged on the rank that owns that slice
    buckets[1][n_slice + 5] = float("nan")
    st2 = [torch.zeros(2, device="cuda") for _ in range(W)]
    vr.reduce_scatter(off, n_slice, dsts, stats=st2, do_stats=True)
    torch.cuda.synchronize()
    assert st2[1][1].item() == 1.0 and st2[0][1].item() == 0.0
    assert native.read_status() == (0, 0)
    vr.close()


@pytest.mark.parametrize("W", [2, 8])
def test_virtual_ranks_reduce_scatter_in_sub_bucket_ranges(W):
    """A bucket reduced in three element ranges (each rank takes what falls into its slice, possibly nothing)
    gives the result and the statistics of the one-launch reduce-scatter."""
    from create_llm_by_cupy_b200.parallel.symm import LocalVirtualRanks

    vr = LocalVirtualRanks(W)
    n_slice = 8 * 700
    n = n_slice * W
    off, buckets = vr.alloc(n, torch.bfloat16)
    for r, b in enumerate(buckets):
        b.copy_(torch.randn(n, generator=torch.Generator().manual_seed(50 + r)).to(torch.bfloat16))
    whole = [torch.zeros(n_slice, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    st_whole = [torch.zeros(2, device="cuda") for _ in range(W)]
    vr.reduce_scatter(off, n_slice, whole, stats=st_whole, do_stats=True)
    parts = [torch.zeros(n_slice, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    st_parts = [torch.zeros(2, device="cuda") for _ in range(W)]
    cuts = [0, 8 * 333, n_slice + 8 * 17, n]          # ranges that start and end inside slices
    for lo, hi in reversed(list(zip(cuts[:-1], cuts[1:]))):     # any order
        vr.reduce_scatter(off, n_slice, parts, stats=st_parts, do_stats=True, elem_range=(lo, hi))
    torch.cuda.synchronize()
    assert native.read_status() == (0, 0)
    for r in range(W):
        assert torch.equal(parts[r], whole[r])
        assert abs(st_parts[r][0].item() - st_whole[r][0].item()) <= 1e-4 * st_whole[r][0].item()
    vr.close()


@pytest.mark.parametrize("W", [2, 4, 8])
def test_virtual_ranks_copy_engine_reduce_scatter_equals_the_pull_kernel(W):
    """The staged form (copy-engine transfers of the peers' parts into local memory, then the summing kernel
    on local memory only) gives the bits and the statistics of the pull kernel: whole bucket, element
    ranges, bf16 store and fp32 accumulation."""
    from create_llm_by_cupy_b200.parallel.symm import LocalVirtualRanks

    vr = LocalVirtualRanks(W)
    n_slice = 8 * 900 + 8
    n = n_slice * W
    off, buckets = vr.alloc(n, torch.bfloat16)
    for r, b in enumerate(buckets):
        b.copy_(torch.randn(n, generator=torch.Generator().manual_seed(70 + r)).to(torch.bfloat16))
    pull = [torch.zeros(n_slice, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    st_pull = [torch.zeros(2, device="cuda") for _ in range(W)]
    vr.reduce_scatter(off, n_slice, pull, stats=st_pull, do_stats=True)
    staged = [torch.zeros(n_slice, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    st_staged = [torch.zeros(2, device="cuda") for _ in range(W)]
    vr.reduce_scatter_staged(off, n_slice, staged, stats=st_staged, do_stats=True)
    parts = [torch.zeros(n_slice, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    cuts = [0, 8 * 411, n_slice + 8 * 23, n]
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        vr.reduce_scatter_staged(off, n_slice, parts, elem_range=(lo, hi))
    acc_pull = [torch.ones(n_slice, device="cuda") for _ in range(W)]
    acc_staged = [torch.ones(n_slice, device="cuda") for _ in range(W)]
    vr.reduce_scatter(off, n_slice, acc_pull, accumulate=True)
    vr.reduce_scatter_staged(off, n_slice, acc_staged, accumulate=True)
    torch.cuda.synchronize()
    assert native.read_status() == (0, 0)
    for r in range(W):
        assert torch.equal(staged[r], pull[r]) and torch.equal(parts[r], pull[r])
        assert torch.equal(acc_staged[r], acc_pull[r])
        assert abs(st_staged[r][0].item() - st_pull[r][0].item()) <= 1e-4 * st_pull[r][0].item()
    vr.close()


def test_virtual_ranks_fused_adam_matches_separate_kernels():
    from create_llm_by_cupy_b200.ops import functional as F
    from create_llm_by_cupy_b200.parallel.symm import LocalVirtualRanks

    W, n_slice = 4, 8 * 500
    vr = LocalVirtualRanks(W)
    off, buckets = vr.alloc(n_slice * W, torch.bfloat16)
    for r, b in enumerate(buckets):
        b.copy_(torch.randn(n_slice * W, generator=torch.Generator().manual_seed(10 + r)).to(torch.bfloat16))
    full = torch.stack([b.float() for b in buckets]).sum(0)
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-6, weight_decay=0.1)
    st = dict(m=[], v=[], master=[], param=[])
    ref = []
    for r in range(W):
        w0 = torch.randn(n_slice, device="cuda", generator=torch.Generator(device="cuda").manual_seed(r))
        st["m"].append(torch.zeros(n_slice, device="cuda"))
        st["v"].append(torch.zeros(n_slice, device="cuda"))
        st["master"].append(w0.clone())
        st["param"].append(torch.zeros(n_slice, dtype=torch.bfloat16, device="cuda"))
        m, v, w, p = torch.zeros(n_slice, device="cuda"), torch.zeros(n_slice, device="cuda"), w0.clone(), \
            torch.zeros(n_slice, dtype=torch.bfloat16, device="cuda")
        F.adamw_step(full[r * n_slice:(r + 1) * n_slice].contiguous(), m, v, w, p, step=1, grad_scale=0.25, **hp)
        ref.append((w, p))
    adam = dict(st, lr=hp["lr"], beta1=hp["beta1"], beta2=hp["beta2"], eps=hp["eps"], weight_decay=hp["weight_decay"],
                m_corr=1 / (1 - 0.9), v_corr=1 / (1 - 0.95), grad_scale=0.25)
    dummy = [torch.empty(8, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    vr.reduce_scatter(off, n_slice, dummy, adam=adam)
    torch.cuda.synchronize()
    assert native.read_status() == (0, 0)
    for r in range(W):
        assert (st["master"][r] - ref[r][0]).abs().max().item() < 1e-5
        assert (st["param"][r].float() - ref[r][1].float()).abs().max().item() < 1e-2
    vr.close()


def test_virtual_ranks_all_gather_and_barrier():
    from create_llm_by_cupy_b200.parallel.symm import LocalVirtualRanks

    W, n = 4, 8 * 333
    vr = LocalVirtualRanks(W)
    off, shards = vr.alloc(n, torch.bfloat16)
    for r, s in enumerate(shards):
        s.copy_(torch.full((n,), float(r + 1)).to(torch.bfloat16))
    outs = [torch.zeros(n * W, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    vr.barrier()
    vr.all_gather(off, n, outs)
    vr.barrier()
    torch.cuda.synchronize()
    ref = torch.cat([torch.full((n,), float(r + 1)) for r in range(W)])
    for o in outs:
        assert torch.equal(o.float().cpu(), ref)
    assert native.read_status() == (0, 0)
    vr.close()


@pytest.mark.parametrize("W,only_b", [(2, False), (4, False), (4, True), (8, True)])
def test_virtual_ranks_gemm_with_the_all_gather_fused_in(W, only_b):
    """One rank's fused all-gather GEMM with all "peer" slices on this device: the unit buffer ends up equal
    to the concatenation of the slices and the product equals the GEMM on the gathered weight - for the form
    that copies the whole unit and the one that copies only the chunks of its own weight."""
    from create_llm_by_cupy_b200.ops import functional as F
    from create_llm_by_cupy_b200.parallel.symm import LocalVirtualRanks

    H, N2, M = 512, 768, 384                          # weight [H, N2] at the start of the unit, then other parameters
    extra = 40_000
    n_unit = ((H * N2 + extra + W * 128 - 1) // (W * 128)) * (W * 128)
    n_slice = n_unit // W
    vr = LocalVirtualRanks(W, heap_bytes=32 << 20)
    off, shards = vr.alloc(n_slice, torch.bfloat16)
    full = (torch.randn(n_unit, generator=torch.Generator().manual_seed(W)) * 0.5).to(torch.bfloat16)
    for r, sh in enumerate(shards):
        sh.copy_(full[r * n_slice:(r + 1) * n_slice])
    a = (torch.randn(M, H, generator=torch.Generator().manual_seed(7)) * 0.5).to(torch.bfloat16).cuda()
    unit_buf = torch.zeros(n_unit, dtype=torch.bfloat16, device="cuda")
    out = vr.gemm_allgather(a, off, n_slice, unit_buf, 0, (H, N2), trans_b=False, only_b=only_b)
    torch.cuda.synchronize()
    assert native.read_status() == (0, 0)
    assert torch.equal(unit_buf.cpu(), full)
    ref = F.gemm(a, full[:H * N2].view(H, N2).cuda())
    assert torch.equal(out, ref)
    vr.close()


def test_heap_guard_blocks_report_a_write_past_the_end_of_an_allocation():
    from create_llm_by_cupy_b200.parallel.comm import SingleProcessComm
    from create_llm_by_cupy_b200.parallel.symm import SymmetricHeap

    heap = SymmetricHeap(SingleProcessComm(), "cuda", heap_bytes=8 << 20)
    a = heap.alloc(1000, torch.bfloat16)
    b = heap.alloc(4096, torch.float32)
    a.fill_(1.0)
    b.fill_(2.0)
    assert heap.check_canaries() == []
    off_b, nbytes_b = heap.guards[1]
    heap.bytes_view[off_b + nbytes_b + 3] = 0          # one byte behind the second allocation
    assert heap.check_canaries() == [1]
    heap.bytes_view[off_b - 1] = 7                     # and one in front of it
    assert heap.check_canaries() == [1]
    with pytest.raises(RuntimeError, match="guard blocks"):
        heap.close()


def test_wait_on_a_flag_nobody_sets_times_out_with_an_error_status():
    """Failure detection on the device: the wait gives up after its (short) budget, records
    ERR_PEER_TIMEOUT and returns; the context stays usable."""
    lib = native.lib()
    native.status_tensor()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    import ctypes
    native.check(lib.b200_symm_wait_probe(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint(1),
                                          ctypes.c_ulonglong(50_000_000), native.stream_ptr()), "wait_probe")
    torch.cuda.synchronize()
    code, kid = native.read_status()
    assert (code, kid) == (2, 204)
    assert native.read_status() == (0, 0)           # cleared, and the device still answers
    x = torch.ones(16, device="cuda")
    assert float(x.sum()) == 16.0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("gather,reduce", [("copy", "pull"), ("gemm", "pull"), ("copy", "copy")])
def test_two_gpu_fused_training_matches_nccl_baseline(tmp_path, gather, reduce):
    """Gradient accumulation over two micro-batches; parameters gathered by the copy engines or inside
    the first consuming GEMM; gradients reduced by the pull kernel or by copy engines + the local kernel."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", B200_TEST_GATHER=gather,
               B200_TEST_REDUCE=reduce, B200_TEST_COPY_MIN="0" if reduce == "copy" else str(1 << 20))
    script = os.path.join(os.path.dirname(__file__), "multi_gpu_worker.py")
    outs = {}
    for mode in ("nccl", "fused"):
        out = tmp_path / f"{mode}.pt"
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
               "--master-addr", "127.0.0.1", "--master-port", str(29600 + (os.getpid() % 300) + (mode == "fused")),
               script, mode, str(out)]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        outs[mode] = torch.load(out)
    a, b = outs["nccl"], outs["fused"]
    for la, lb in zip(a["losses"], b["losses"]):
        assert abs(la - lb) < 3e-2, (a["losses"], b["losses"])
    assert abs(a["param_norm"] - b["param_norm"]) < 1e-2 * a["param_norm"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_fused_reduce_scatter_adam_matches_nccl_baseline(tmp_path):
    """Reduce-scatter + AdamW in one kernel per unit (no clipping) against NCCL + separate AdamW."""
    script = os.path.join(os.path.dirname(__file__), "multi_gpu_worker.py")
    outs = {}
    for mode, extra in (("nccl", {"B200_TEST_NOCLIP": "1"}), ("fused", {"B200_TEST_FUSED_ADAM": "1"})):
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", B200_TEST_ACCUM="1",
                   B200_TEST_GATHER="pull", **extra)
        out = tmp_path / f"{mode}.pt"
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
               "--master-addr", "127.0.0.1", "--master-port", str(29700 + (os.getpid() % 200) + (mode == "fused")),
               script, mode, str(out)]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        outs[mode] = torch.load(out)
    for la, lb in zip(outs["nccl"]["losses"], outs["fused"]["losses"]):
        assert abs(la - lb) < 3e-2, (outs["nccl"]["losses"], outs["fused"]["losses"])
    assert abs(outs["nccl"]["param_norm"] - outs["fused"]["param_norm"]) < 1e-2 * outs["nccl"]["param_norm"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("zero,ratio", [("3", 0.0), ("2.5", 0.5)])
def test_launcher_trains_on_the_fused_collectives_by_default_and_matches_nccl(tmp_path, zero, ratio):
    """``TrainMultiGPU`` (the product entry path) on 2 GPUs: by default the peer-memory collectives carry the
    data plane (their launch and copy-engine counters move), and the loss curve equals that of the NCCL
    run. ZeRO-2.5: the replica gradients and the replica rebuild take the same kernels."""
    from create_llm_by_cupy_b200.parallel.trainer import TrainMultiGPU, TrainMultiGPU_ZeRO25
    from create_llm_by_cupy_b200.utils import checkpoint as ckpt

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    md = dict(vocab_size=2048, hidden_size=256, layer_num=3, time_size=256, q_head=4, kv_head=2, ffn_size=768,
              padding_id=0, dropout_rate=0, dtype="bf16", half_float=True, tie_embeddings=True, init_std=0.02, seed=1,
              zero3_gather_mode="copy", zero3_copy_min_bytes=0)
    cls = TrainMultiGPU_ZeRO25 if zero == "2.5" else TrainMultiGPU
    res = {}
    for k, mode in enumerate(("fused", "nccl")):
        out = tmp_path / mode
        kw = dict(zero25_replica_ratio=ratio) if zero == "2.5" else {}
        codes = None
        for attempt in range(2):      # one more try when a worker process did not come up (a port, an NCCL bootstrap)
            launcher = cls(dict(md, zero3_fused_collectives=mode == "fused"), use_devices=[0, 1], batch_size=2,
                           accum_step=1, console=False, result_dir=str(out), synthetic_samples=64, lr_max=1e-3,
                           warm_up=1, beta2=0.95, peer_wait_s=10.0, collective_timeout_s=120.0,
                           heartbeat_timeout_s=300.0,
                           master_port=24000 + (os.getpid() % 2000) + 7 * k + (50 if zero == "2.5" else 0) + 100 * attempt,
                           **kw)
            try:
                codes = launcher.fit(2 * 2 * 6)
            except Exception as e:      # WorkerFailure: a rank exited with an error or stopped answering
                codes = None
                print(f"launcher attempt {attempt} failed: {e}", file=sys.stderr)
                if attempt == 1:
                    raise
            if codes == [0, 0]:
                break
        assert codes == [0, 0]
        res[mode] = ckpt.read_pickle_gzip(str(out / "result_rank0.pkl.gz"))
    f, n = res["fused"], res["nccl"]
    assert f["collectives"] == "fused:copy" and n["collectives"] == "nccl"
    assert f["fused_launches"] > 0 and f["copy_engine_transfers"] > 0 and n["fused_launches"] == 0
    assert len(f["losses"]) == 6
    for la, lb in zip(f["losses"], n["losses"]):
        assert abs(la - lb) < 3e-2, (f["losses"], n["losses"])
