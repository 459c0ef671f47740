"""Micro-benchmark of the peer-memory collectives against NCCL, on the ZeRO unit of one 1.3 B block.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port P bench_collectives.py [--json out.json]
    python bench_collectives.py --virtual 4        # one GPU, W virtual ranks in one launch (for ncu)

The unit is what the training step moves per transformer block: 45.1 M bf16 parameters (K|Q|V, O,
gate|value and down projections of d_model 2048 / FFN 5504), padded to a multiple of 128 W elements.
Timed with CUDA events (3 warm-up calls, median of 7, max over ranks, a 256 MB buffer written between
calls so that nothing is served from L2):

  reduce_scatter  fused kernel (pull every peer's slice of the gradient bucket, fp32 sum, bf16 store,
                  sum of squares and non-finite flag) against ncclReduceScatter + the separate
                  statistics kernel; reduce_scatter_copy_engine: the peers' parts are brought into local
                  memory by the copy engines between two barriers and the same kernel sums local memory;
  rs_adam         the same kernel in its AdamW mode (reduced gradient never stored) against
                  ncclReduceScatter + statistics + AdamW kernels;
  all_gather      copy engines (one cudaMemcpyAsync per peer slice, no SM) and the pull kernel against
                  ncclAllGather;
  ag_gemm         K|Q|V projection of 8192 tokens with the gather done inside the GEMM - the whole unit,
                  or (the form the training step uses) only the chunks that hold K|Q|V while the
                  stand-alone kernel pulls the rest of the unit on another stream - against
                  ncclAllGather followed by the GEMM.

Every rank receives (W - 1) / W of the unit over NVLink in each of these, so the bound is that many
bytes over the measured peer-copy bandwidth (770 GB/s per direction); ``of_link`` is achieved / bound.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from create_llm_by_cupy_b200.ops import functional as F  # noqa: E402
from create_llm_by_cupy_b200.ops import native  # noqa: E402
from create_llm_by_cupy_b200.ops.gemm import ag_region, gemm, gemm_allgather  # noqa: E402

LINK_GBS = 770.0
H, NKQV, I, M = 2048, 3072, 5504, 8192
SIZES = [H * NKQV, H * H, H * 2 * I, I * H]


def median_ms(fn, flush, sync, iters=7, warm=3):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def run_virtual(W: int):
    """All W ranks in one launch on one GPU: peer traffic is local HBM traffic, so this mode is for
    counters (ncu) and correctness, not for link bandwidth."""
    from create_llm_by_cupy_b200.parallel.symm import LocalVirtualRanks
    total = sum(SIZES)
    pad = (total + W * 128 - 1) // (W * 128) * (W * 128)
    n = pad // W
    vr = LocalVirtualRanks(W, "cuda", heap_bytes=(pad * 2 + n * 2 + (1 << 20)) + (64 << 10))
    boff, buckets = vr.alloc(pad, torch.bfloat16)
    soff, shards = vr.alloc(n, torch.bfloat16)
    for r in range(W):
        buckets[r].normal_(0, 0.02)
        shards[r].normal_(0, 0.02)
    dsts = [torch.empty(n, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    outs = [torch.empty(pad, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    stats = [torch.zeros(2, device="cuda") for _ in range(W)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    sync = torch.cuda.synchronize
    rs = median_ms(lambda: vr.reduce_scatter(boff, n, dsts, stats=stats, do_stats=True, blocks=64 // W), flush, sync)
    ag = median_ms(lambda: vr.all_gather(soff, n, outs, blocks=64 // W), flush, sync)
    # the copy form as ONE rank runs it: W - 1 device-to-device copies into the staging buffer, then the summing kernel
    # on local memory (2 CTAs per SM)
    stage = torch.empty(n * max(W - 1, 1), dtype=torch.bfloat16, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rs_staged = median_ms(lambda: vr.reduce_scatter_staged(boff, n, dsts, stats=stats, do_stats=True, blocks=2 * sms,
                                                           ranks=[0], stage=stage), flush, sync)
    ref = sum(b.float().view(W, n)[0] for b in buckets)
    err = (dsts[0].float() - ref).abs().max().item()
    print(json.dumps({"mode": f"virtual{W}", "unit_bytes": pad * 2, "reduce_scatter_ms": rs, "all_gather_ms": ag,
                      "reduce_scatter_staged_one_rank_ms": rs_staged,
                      "rs_max_err": err, "status": native.read_status()}))
    vr.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--virtual", type=int, default=0)
    ap.add_argument("--parallel-copies", action="store_true", help="peer copies side by side on helper streams (A/B)")
    ap.add_argument("--blocks", type=int, default=0, help="CTAs of the fused collective kernels (0: default)")
    args = ap.parse_args()
    if args.virtual:
        return run_virtual(args.virtual)
    from create_llm_by_cupy_b200.parallel.comm import init_distributed, shutdown_distributed
    from create_llm_by_cupy_b200.parallel.symm import FusedCollectives
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = init_distributed(rank, world, backend="nccl", device_id=local, master_port=int(os.environ["MASTER_PORT"]))
    kw = dict(rs_blocks=args.blocks, ag_blocks=args.blocks) if args.blocks > 0 else {}
    fc = FusedCollectives(comm, dev, heap_bytes=2 << 30, **kw)
    if args.parallel_copies:
        fc.lib.b200_symm_parallel_copies(1)
    total = sum(SIZES)
    pad = (total + world * 128 - 1) // (world * 128) * (world * 128)
    n = pad // world
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    bucket = fc.alloc(pad, torch.bfloat16)
    shard = fc.alloc(n, torch.bfloat16)
    bucket.copy_(torch.randn(pad, device=dev, generator=gen).to(torch.bfloat16) * 0.02)
    shard.copy_(torch.randn(n, device=dev, generator=gen).to(torch.bfloat16) * 0.02)
    dst = torch.empty(n, dtype=torch.bfloat16, device=dev)
    dst_ref = torch.empty_like(dst)
    full = torch.empty(pad, dtype=torch.bfloat16, device=dev)
    full_ref = torch.empty_like(full)
    stats, stats_ref = torch.zeros(2, device=dev), torch.zeros(2, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    master = shard.float().clone()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hp = dict(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-6, weight_decay=0.1)

    def sync():
        torch.cuda.synchronize()
        comm.barrier()

    def nccl_rs():
        torch.distributed.reduce_scatter_tensor(dst_ref, bucket)
        F.grad_stats(dst_ref, stats_ref)

    def nccl_rs_adam():
        torch.distributed.reduce_scatter_tensor(dst_ref, bucket)
        F.grad_stats(dst_ref, stats_ref)
        F.adamw_step(dst_ref, m, v, master, shard, step=1, grad_scale=1.0 / world, **hp)

    def gather(copy_engine: bool):
        fc.copy_engine = copy_engine
        fc.all_gather(full, shard)

    def reduce(mode: str):
        fc.reduce_mode = mode
        fc.reduce_scatter_accumulate(dst, bucket, accumulate=False, stats=stats, do_stats=True)

    fc.reserve_stage(n)

    adam = dict(m=m, v=v, master=master, param=shard, m_corr=1.0 / (1 - 0.9), v_corr=1.0 / (1 - 0.95),
                grad_scale=1.0 / world, **hp)
    res = {}
    recv = (world - 1) / world * pad * 2          # bytes every rank receives over NVLink
    bound_ms = recv / (LINK_GBS * 1e9) * 1e3
    cases = [
        ("reduce_scatter", lambda: reduce("pull"), nccl_rs),
        ("reduce_scatter_copy_engine", lambda: reduce("copy"), nccl_rs),
        ("rs_adam", lambda: fc.reduce_scatter_accumulate(dst, bucket, accumulate=False, stats=stats, do_stats=True, adam=adam), nccl_rs_adam),
        ("all_gather_copy_engine", lambda: gather(True), lambda: torch.distributed.all_gather_into_tensor(full_ref, shard)),
        ("all_gather", lambda: gather(False), lambda: torch.distributed.all_gather_into_tensor(full_ref, shard)),
    ]
    for name, fused_fn, nccl_fn in cases:
        t_f = torch.tensor([median_ms(fused_fn, flush, sync)], device=dev)
        t_n = torch.tensor([median_ms(nccl_fn, flush, sync)], device=dev)
        comm.all_reduce(t_f, op="max")
        comm.all_reduce(t_n, op="max")
        res[name] = {"fused_ms": float(t_f), "nccl_ms": float(t_n), "bound_ms": bound_ms,
                     "fused_of_link": bound_ms / float(t_f), "nccl_of_link": bound_ms / float(t_n),
                     "fused_GBs_in": recv / float(t_f) / 1e6}
    # correctness of the plain modes (the AdamW mode has changed `shard` by now: refresh first)
    fc.barrier()
    shard.copy_(torch.randn(n, device=dev, generator=gen).to(torch.bfloat16) * 0.02)
    fc.barrier()
    sync()
    fc.reduce_scatter_accumulate(dst, bucket, accumulate=False, stats=stats, do_stats=False)
    torch.distributed.reduce_scatter_tensor(dst_ref, bucket)
    dst_staged = torch.empty_like(dst)
    fc.reduce_mode = "copy"
    fc.reduce_scatter_accumulate(dst_staged, bucket, accumulate=False, stats=stats, do_stats=False)
    fc.reduce_mode = "pull"
    sync()
    res["rs_copy_engine_equals_pull"] = bool(torch.equal(dst_staged, dst))
    torch.distributed.all_gather_into_tensor(full_ref, shard)
    res["ag_equal_nccl"] = True
    for ce in (True, False):
        full.zero_()
        gather(ce)
        sync()
        res["ag_equal_nccl"] = bool(res["ag_equal_nccl"] and torch.equal(full, full_ref))
    res["rs_max_abs_diff_vs_nccl"] = (dst.float() - dst_ref.float()).abs().max().item()

    # all-gather fused into the K|Q|V projection
    x = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
    peers = [b + fc.heap.offset_of(shard) for b in fc.heap.peer_bases]
    unit = torch.zeros(pad, dtype=torch.bfloat16, device=dev)
    seg = torch.zeros((pad * 2 + (1 << 20) - 1) >> 20, dtype=torch.int64, device=dev)
    out = torch.empty(M, NKQV, dtype=torch.bfloat16, device=dev)
    ep = [0]

    def fused_ag_gemm():
        ep[0] += 1
        gemm_allgather(x, unit, 0, (H, NKQV), trans_b=False, peer_slices=peers, seg=seg, epoch=ep[0], n_copy=fc.n_copy,
                       out=out)

    # the split form used by the training step: the GEMM pulls only the chunks of its own weight, the rest
    # of the unit is pulled by the stand-alone kernel on another stream at the same time
    side = torch.cuda.Stream(device=dev)
    region = ag_region(n * 2, world, 0, H * NKQV * 2)

    def split_ag_gemm(copy_engine: bool = False):
        cur = torch.cuda.current_stream()
        side.wait_stream(cur)
        fc.copy_engine = copy_engine
        fc.all_gather(unit, shard, side, skip=region)
        seg.zero_()
        gemm_allgather(x, unit, 0, (H, NKQV), trans_b=False, peer_slices=peers, seg=seg, epoch=1, n_copy=fc.n_copy,
                       out=out, only_b=True)
        cur.wait_stream(side)

    def nccl_ag_gemm():
        torch.distributed.all_gather_into_tensor(full_ref, shard)
        gemm(x, full_ref[:H * NKQV].view(H, NKQV), out=out)

    gemm_only = median_ms(lambda: gemm(x, full_ref[:H * NKQV].view(H, NKQV), out=out), flush, sync)
    t_f = torch.tensor([median_ms(fused_ag_gemm, flush, sync)], device=dev)
    t_s = torch.tensor([median_ms(split_ag_gemm, flush, sync)], device=dev)
    t_c = torch.tensor([median_ms(lambda: split_ag_gemm(True), flush, sync)], device=dev)
    t_n = torch.tensor([median_ms(nccl_ag_gemm, flush, sync)], device=dev)
    comm.all_reduce(t_c, op="max")
    comm.all_reduce(t_f, op="max")
    comm.all_reduce(t_s, op="max")
    comm.all_reduce(t_n, op="max")
    unit.zero_()
    sync()
    split_ag_gemm()
    torch.distributed.all_gather_into_tensor(full_ref, shard)
    sync()
    res["split_ag_gemm_unit_equal_nccl"] = bool(torch.equal(unit, full_ref))
    unit.zero_()
    sync()
    split_ag_gemm(True)
    sync()
    res["split_ag_gemm_copy_engine_unit_equal_nccl"] = bool(torch.equal(unit, full_ref))
    res["split_ag_gemm_max_err"] = (out.float() - gemm(x, full_ref[:H * NKQV].view(H, NKQV)).float()).abs().max().item()
    peak = 1590.0
    peaks_file = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(peaks_file):
        peak = float(json.load(open(peaks_file)).get("bf16_tflops", peak))
    gemm_bound = 2.0 * M * NKQV * H / (peak * 1e12) * 1e3
    target = max(gemm_bound, bound_ms)
    res["ag_gemm"] = {"whole_unit_in_gemm_ms": float(t_f), "own_weight_in_gemm_rest_pulled_ms": float(t_s),
                      "own_weight_in_gemm_rest_by_copy_engines_ms": float(t_c),
                      "nccl_then_gemm_ms": float(t_n), "gemm_alone_ms": gemm_only,
                      "bound_ms": target, "fused_of_roofline": target / min(float(t_s), float(t_c)),
                      "nccl_then_gemm_of_roofline": target / float(t_n)}
    res["status"] = native.read_status()
    res["world"] = world
    res["blocks"] = fc.rs_blocks
    res["unit_bytes"] = pad * 2
    if rank == 0:
        print(json.dumps(res))
        if args.json:
            with open(args.json, "w") as f:
                json.dump(res, f, indent=1)
    comm.barrier()
    fc.close()
    shutdown_distributed()


if __name__ == "__main__":
    main()
