"""Stand-alone causal GQA flash-attention benchmark (forward + backward with RoPE, base 10000).

Shapes: batch 8, 32 query / 8 KV heads, head_dim 128 (or 64: --head-dim), bf16, seq lengths 1024..16384; Q, K, V, dO
drawn i.i.d. N(0, 1) with seed 0. Two implementations are timed with CUDA events (3 warm-up, then
the median of 5; inputs of every length exceed the 126 MB L2 from T = 4096 up, below that a 256 MB
buffer is written between iterations):

  tcgen05 : rotary embedding applied in place to Q and K (one elementwise pass, included in the
            time), tcgen05/TMEM forward, dK/dV and dQ kernels, inverse rotation of dQ and dK (in the
            kernels' epilogues where that form exists, else one more pass);
  mma     : the mma.sync kernels with the rotation fused into their tile loads.

FLOPs counted: 4*B*H*T^2*D/2 forward, 2.5x that backward (the usual 5-GEMM convention; the
kernels here recompute S and dP in both backward kernels, which is not counted).

    python bench_flash.py [--seqs 1024,2048,...] [--head-dim 128] [--json out.json]
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


def timed(fn, flush, iters=5, warm=3):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", default="1024,2048,4096,8192,16384")
    ap.add_argument("--json", default=None)
    ap.add_argument("--head-dim", type=int, default=128, choices=(64, 128))
    a = ap.parse_args()
    dev = "cuda"
    B, QH, KVH, D = 8, 32, 8, a.head_dim
    peak = 1648.3
    try:
        peak = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:
        pass
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for T in [int(v) for v in a.seqs.split(",")]:
        g = torch.Generator(device=dev).manual_seed(0)
        packed = torch.randn(B * T, (QH + 2 * KVH) * D, device=dev, generator=g).to(torch.bfloat16)
        do = torch.randn(B, T, QH, D, device=dev, generator=g).to(torch.bfloat16)
        tabs = F.rope_table(T, D, 10000.0, dev)
        v3 = packed.view(B, T, -1)
        k = v3[:, :, :KVH * D].unflatten(2, (KVH, D))
        q = v3[:, :, KVH * D:(KVH + QH) * D].unflatten(2, (QH, D))
        v = v3[:, :, (KVH + QH) * D:].unflatten(2, (KVH, D))
        dpacked = torch.empty_like(packed)
        d3 = dpacked.view(B, T, -1)
        dk = d3[:, :, :KVH * D].unflatten(2, (KVH, D))
        dq = d3[:, :, KVH * D:(KVH + QH) * D].unflatten(2, (QH, D))
        dv = d3[:, :, (KVH + QH) * D:].unflatten(2, (KVH, D))
        fl_f = 4.0 * B * QH * T * T * D / 2
        res = {"T": T}
        for impl in ("tcgen05", "mma"):
            st = {}

            def fwd():
                if impl == "tcgen05":
                    F.FLASH_TC = True
                    F.rope_inplace(packed, tabs[0], tabs[1], T, KVH + QH, D, col0=0)
                    st["o"], st["lse"] = F.flash_attn_fwd(q, k, v, rope=None)
                else:
                    F.FLASH_TC = False
                    st["o"], st["lse"] = F.flash_attn_fwd(q, k, v, rope=tabs)

            def bwd():
                if impl == "tcgen05":
                    F.FLASH_TC = True
                    fused = F.flash_bwd_can_unrotate(q)
                    F.flash_attn_bwd(do, q, k, v, st["o"], st["lse"], rope=None, out=(dq, dk, dv),
                                     unrotate=tabs if fused else None)
                    if not fused:
                        F.rope_inplace(dpacked, tabs[0], tabs[1], T, KVH + QH, D, col0=0, inverse=True)
                else:
                    F.FLASH_TC = False
                    F.flash_attn_bwd(do, q, k, v, st["o"], st["lse"], rope=tabs, out=(dq, dk, dv))

            fl = flush if T < 4096 else None
            tf = timed(fwd, fl)
            tb = timed(bwd, fl)
            res[impl] = {"fwd_ms": tf, "bwd_ms": tb, "fwd_tflops": fl_f / tf / 1e9, "bwd_tflops": 2.5 * fl_f / tb / 1e9,
                         "fwd_bwd_tflops": 3.5 * fl_f / (tf + tb) / 1e9,
                         "fraction_of_measured_bf16_peak": 3.5 * fl_f / (tf + tb) / 1e9 / peak}
        native.raise_on_status()
        rows.append(res)
        print(json.dumps(res), flush=True)
        del packed, do, dpacked
    F.FLASH_TC = True
    if a.json:
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
