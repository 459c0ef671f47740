"""GEMM micro-benchmark: the tcgen05 kernel against torch.matmul (cuBLAS) on one shape.

    python bench_gemm.py --m 8192 --n 3072 --k 2048 --layout nn --iters 20

layout: nn = x @ W (W [K, N]), nt = x @ W^T (W [N, K]), tn = x^T @ dy (x [K, M]). A 256 MB buffer is
written between timed iterations so operands come from HBM, not L2. With --iters 1 --no-ref the
script launches the kernel exactly (warm + 1) times, which is the form used under ncu.

--epilogue selects a fused form of the CTA-pair kernel and times it against the kernels it replaces:
  swiglu      gate|value projection (N = 2 I) leaving silu(gate) * value and the raw projection,
              against the GEMM followed by the activation kernel (--n is I);
  swiglu_bwd  down-projection dgrad (x @ W_out^T, N = I, K = H) whose epilogue turns d(act) into d(gate|value),
              against the GEMM followed by the activation-backward kernel;
  delta       output-projection dgrad (dY @ W_O^T, N = heads x 128, rows = batch x 2048) whose epilogue also leaves the
              attention backward's delta = rowsum(dO * O), against the GEMM followed by the delta kernel;
  ce          LM head (x @ W^T, N = vocabulary): statistics epilogue (no logits stored) plus merge, then the
              logit-gradient epilogue, against fp32 logits + row-statistics kernel + logit-gradient kernel.
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


def _timer(a):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

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
    return run


def fused_epilogue(a):
    from create_llm_by_cupy_b200.ops import functional as F
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    run = _timer(a)
    M, N, K = a.m, a.n, a.k
    res = {"epilogue": a.epilogue, "m": M, "n": N, "k": K}
    if a.epilogue == "swiglu":
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(K, 2 * N, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        fl = 2.0 * M * 2 * N * K
        t = run(lambda: F.gemm_swiglu(x, w, keep_gv=True))
        res.update(fused_ms=t, fused_tflops=fl / t / 1e9)
        if not a.no_ref:
            t2 = run(lambda: F.swiglu_fwd(gemm(x, w)))
            res.update(separate_ms=t2, separate_tflops=fl / t2 / 1e9)
    elif a.epilogue == "swiglu_bwd":
        dout = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        w_out = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        gv = torch.randn(M, 2 * N, device=dev, generator=g).to(torch.bfloat16)
        fl = 2.0 * M * N * K
        t = run(lambda: F.gemm_swiglu_bwd(dout, w_out, gv))
        res.update(fused_ms=t, fused_tflops=fl / t / 1e9)
        if not a.no_ref:
            t2 = run(lambda: F.swiglu_bwd(gemm(dout, w_out, trans_b=True), gv))
            res.update(separate_ms=t2, separate_tflops=fl / t2 / 1e9)
    elif a.epilogue == "delta":
        T, D = 2048, 128
        assert M % T == 0 and N % D == 0
        dy = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        w_o = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        o = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
        fl = 2.0 * M * N * K
        t = run(lambda: F.gemm_delta(dy, w_o, o, T, D))
        res.update(fused_ms=t, fused_tflops=fl / t / 1e9)
        if not a.no_ref:
            o4 = o.view(M // T, T, N // D, D)
            dl = torch.empty(M // T, N // D, T, device=dev)

            def sep():
                do = gemm(dy, w_o, trans_b=True)
                F.flash_delta(o4, do.view_as(o4), dl)
            t2 = run(sep)
            res.update(separate_ms=t2, separate_tflops=fl / t2 / 1e9)
    else:
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        t_ids = torch.randint(1, N, (M,), device=dev, generator=g, dtype=torch.int32)
        tl = torch.zeros(M, device=dev)
        fl = 2.0 * M * N * K
        chunk = 8192

        def fwd_fused():
            pmax, psum = F.gemm_ce_stats(x, w, t_ids, tl, vocab=N)
            return F.ce_merge(pmax, psum)

        rmax, rsum = fwd_fused()
        cnt = F.ce_loss(rmax, rsum, tl, t_ids, 0)
        lse, coef = F.ce_row_coef(rmax, rsum, t_ids, cnt, 0, 1.0)

        def bwd_fused():
            for s0 in range(0, N, chunk):
                F.gemm_ce_dlogits(x, w[s0:min(s0 + chunk, N)], t_ids, lse, coef, col0=s0)

        def fwd_sep():
            rm, rs = torch.empty(M, device=dev), torch.empty(M, device=dev)
            for i, s0 in enumerate(range(0, N, chunk)):
                lg = gemm(x, w[s0:min(s0 + chunk, N)], trans_b=True, out_dtype=torch.float32)
                F.ce_stats(lg, t_ids, rm, rs, tl, s0, i == 0)

        def bwd_sep():
            for s0 in range(0, N, chunk):
                lg = gemm(x, w[s0:min(s0 + chunk, N)], trans_b=True, out_dtype=torch.float32)
                F.ce_dlogits(lg, t_ids, rmax, rsum, cnt, s0, 0, 1.0, torch.bfloat16)

        tf, tb = run(fwd_fused), run(bwd_fused)
        res.update(fused_fwd_ms=tf, fused_fwd_tflops=fl / tf / 1e9, fused_dlogits_ms=tb, fused_dlogits_tflops=fl / tb / 1e9)
        if not a.no_ref:
            res.update(separate_fwd_ms=run(fwd_sep), separate_dlogits_ms=run(bwd_sep))
    native.raise_on_status()
    print(json.dumps(res))


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
    ap.add_argument("--epilogue", default="none", choices=["none", "swiglu", "swiglu_bwd", "delta", "ce"])
    a = ap.parse_args()
    dev = "cuda"
    if a.epilogue != "none":
        return fused_epilogue(a)
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
