"""GEMM micro-benchmark: the tcgen05 kernel against torch.matmul (cuBLAS) on one shape.

    python bench_gemm.py --m 8192 --n 3072 --k 2048 --layout nn --iters 20

layout: nn = x @ W (W [K, N]), nt = x @ W^T (W [N, K]), tn = x^T @ dy (x [K, M]). A 256 MB buffer is
written between timed iterations so operands come from HBM, not L2. With --iters 1 --no-ref the
script launches the kernel exactly (warm + 1) times, which is the form used under ncu.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from create_llm_by_cupy_b200.ops import native  # noqa: E402
from create_llm_by_cupy_b200.ops.gemm import gemm  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--layout", default="nn", choices=["nn", "nt", "tn"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warm", type=int, default=2)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--no-ref", action="store_true")
    a = ap.parse_args()
    dev = "cuda"
    ta, tb = a.layout[0] == "t", a.layout[1] == "t"
    g = torch.Generator(device=dev).manual_seed(0)
    A = torch.randn((a.k, a.m) if ta else (a.m, a.k), device=dev, generator=g).to(torch.bfloat16)
    B = torch.randn((a.n, a.k) if tb else (a.k, a.n), device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def run(fn):
        for _ in range(a.warm):
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]

    fl = 2.0 * a.m * a.n * a.k
    t = run(lambda: gemm(A, B, trans_a=ta, trans_b=tb, out=out, bn=a.bn))
    res = {"m": a.m, "n": a.n, "k": a.k, "layout": a.layout, "ms": t, "tflops": fl / t / 1e9}
    if not a.no_ref:
        At, Bt = (A.t() if ta else A), (B.t() if tb else B)
        t2 = run(lambda: torch.matmul(At, Bt, out=out))
        res.update({"cublas_ms": t2, "cublas_tflops": fl / t2 / 1e9})
    native.raise_on_status()
    print(json.dumps(res))


if __name__ == "__main__":
    main()
