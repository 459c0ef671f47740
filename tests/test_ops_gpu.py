"""Numerics of every native kernel against the fp32 PyTorch restatement of the same op.

The reference of each op is the CPU body of the same front-end function, fed fp32 copies of the
bf16 inputs, so the comparison isolates the kernel (not input rounding).
"""
import math

import pytest
import torch

from create_llm_by_cupy_b200.ops import functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def close(a, b, rtol=2e-2, atol=2e-2, frob=1e-2):
    """Two bounds: the maximum error against the tensor's scale, and the relative Frobenius error - the
    second one catches a wrong tile of small values that the first lets through."""
    a = a.float().cpu()
    b = b.float().cpu()
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin), "non-finite entries differ"
    a, b = a[fin], b[fin]
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"max err {err} vs ref scale {ref}"
    if frob is not None and b.numel() > 1:
        rel = ((a - b).norm() / (b.norm() + 1e-20)).item()
        assert rel <= frob, f"relative Frobenius error {rel} > {frob}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 328, 136), (1000, 520, 264), (72, 40, 8), (64, 100, 33)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm(M, N, K, ta, tb):
    a = bf(*((K, M) if ta else (M, K)), seed=1)
    b = bf(*((N, K) if tb else (K, N)), seed=2)
    ref = F.gemm(a.float(), b.float(), trans_a=ta, trans_b=tb)
    for impl in ("1cta", "2cta"):
        out = F.gemm(a.to(DEV), b.to(DEV), trans_a=ta, trans_b=tb, impl=impl)
        close(out, ref, rtol=1e-2, atol=1e-2)
    assert F.native.read_status() == (0, 0)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 520, 264), (1000, 1032, 136), (2048, 768, 512)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_cta_pairs(M, N, K, ta, tb):
    """cta_group::2 kernel: 256 x 256 tiles over two SMs, ragged edges, accumulate epilogue."""
    a = bf(*((K, M) if ta else (M, K)), seed=3)
    b = bf(*((N, K) if tb else (K, N)), seed=4)
    c = bf(M, N, seed=5)
    ref = F.gemm(a.float(), b.float(), trans_a=ta, trans_b=tb) + c.float()
    out = F.gemm(a.to(DEV), b.to(DEV), trans_a=ta, trans_b=tb, add=c.to(DEV), impl="2cta")
    close(out, ref, rtol=1e-2, atol=1e-2)
    assert F.native.read_status() == (0, 0)


@pytest.mark.parametrize("M,N,K,ta,tb,mode", [
    (8192, 2048, 128, False, False, "plain"),      # 256 tiles on 74 pairs: the last 34 are run as 68 half tiles
    (8192, 2048, 192, False, True, "add"),
    (2048, 3072, 256, True, False, "plain"),       # 96 tiles: 22 of them halved
    (2048, 3000, 128, True, False, "fp32"),        # ragged last column tile, fp32 output
    (4864, 4104, 64, False, True, "add"),          # 19 x 17 = 323 tiles (27 left over), ragged N
])
def test_gemm_cta_pairs_half_tiles(M, N, K, ta, tb, mode):
    """Shapes with more tiles than CTA pairs whose last round is less than half full: those tiles are
    computed as 256 x 128 halves. Checked against fp32 on the device (the matrices are large)."""
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    a = torch.randn((K, M) if ta else (M, K), device=DEV, generator=g).to(torch.bfloat16)
    b = torch.randn((N, K) if tb else (K, N), device=DEV, generator=g).to(torch.bfloat16)
    ref = (a.float().t() if ta else a.float()) @ (b.float().t() if tb else b.float())
    if mode == "add":
        c = torch.randn(M, N, device=DEV, generator=g).to(torch.bfloat16)
        out = F.gemm(a, b, trans_a=ta, trans_b=tb, add=c, impl="2cta")
        ref = ref + c.float()
    elif mode == "fp32":
        out = F.gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32, impl="2cta")
    else:
        out = F.gemm(a, b, trans_a=ta, trans_b=tb, impl="2cta")
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err


@pytest.mark.parametrize("M,N,K,T,D,rope_cols", [
    (1000, 768, 136, 250, 128, 640),          # ragged M, rotation ends inside a tile
    (8192, 3072, 128, 2048, 128, 2560),       # the 1.3 B projection shape (part of its tiles run as halves)
    (2048, 1280, 192, 1024, 64, 1024),        # 64-wide heads
    (512, 512, 64, 512, 64, 512),
])
def test_gemm_with_rotary_epilogue(M, N, K, T, D, rope_cols):
    """gemm_rope = GEMM followed by the in-place rotary pass over the first rope_cols columns."""
    g = torch.Generator(device=DEV).manual_seed(M + N)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    b = (torch.randn(K, N, device=DEV, generator=g) * 0.1).to(torch.bfloat16)
    cos, sin = F.rope_table(T, D, 10000.0, DEV)
    assert F.gemm_rope_fusable(a, b, D, rope_cols)
    out = F.gemm_rope(a, b, cos, sin, T, D, rope_cols)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    ref = (a.float() @ b.float()).cpu()
    F.rope_inplace(ref, cos.cpu(), sin.cpu(), T, rope_cols // D, D, col0=0)
    close(out, ref, rtol=1e-2, atol=2e-2)
    two_step = F.gemm(a, b)
    F.rope_inplace(two_step, cos, sin, T, rope_cols // D, D, col0=0)
    close(out, two_step, rtol=1e-2, atol=2e-2)
    assert torch.equal(out[:, rope_cols:], F.gemm(a, b)[:, rope_cols:])


@pytest.mark.parametrize("M,I,K", [(256, 128, 64), (300, 688, 264), (1000, 1376, 136), (2048, 5504, 256), (512, 200, 72)])
@pytest.mark.parametrize("keep_gv", [True, False])
def test_gemm_with_swiglu_epilogue(M, I, K, keep_gv):
    """gate|value projection with the activation in the GEMM epilogue (ragged I: the last tile's gate columns run
    into the value half and must be clipped; I = 200 puts a whole 64-column group past the edge)."""
    x = bf(M, K, seed=21)
    w = bf(K, 2 * I, scale=0.3, seed=22)
    assert F.gemm_swiglu_fusable(x.to(DEV), w.to(DEV))
    gv_ref = x.float() @ w.float()
    act_ref = torch.nn.functional.silu(gv_ref[:, :I]) * gv_ref[:, I:]
    canary = torch.full((M + 2, 2 * I), 7.0, dtype=torch.bfloat16, device=DEV)
    gv, act = F.gemm_swiglu(x.to(DEV), w.to(DEV), keep_gv=keep_gv)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    assert (gv is None) == (not keep_gv)
    close(act, act_ref, rtol=1e-2, atol=1e-2)
    if keep_gv:
        close(gv, gv_ref, rtol=1e-2, atol=1e-2)
        # the separate activation kernel on the stored projection agrees up to the bf16 rounding of gv
        close(act, F.swiglu_fwd(gv), rtol=2e-2, atol=2e-2)
    del canary


@pytest.mark.parametrize("M,I,K", [(256, 256, 64), (300, 688, 264), (1000, 1376, 136), (2048, 5504, 256), (512, 328, 72)])
def test_gemm_with_swiglu_backward_epilogue(M, I, K):
    """d(act) = dout W_out^T stays in tensor memory; the epilogue fetches gate / value tiles and writes their
    gradients (ragged I: the last tile is half or mostly past the edge)."""
    dout = bf(M, K, seed=41)
    w_out = bf(I, K, scale=0.3, seed=42)
    gv = bf(M, 2 * I, seed=43)
    assert F.gemm_swiglu_bwd_fusable(dout.to(DEV), w_out.to(DEV), gv.to(DEV))
    dact = dout.float() @ w_out.float().t()
    g, v = gv[:, :I].float(), gv[:, I:].float()
    sg = torch.sigmoid(g)
    ref = torch.cat([dact * v * sg * (1 + g * (1 - sg)), dact * g * sg], 1)
    out = F.gemm_swiglu_bwd(dout.to(DEV), w_out.to(DEV), gv.to(DEV))
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    close(out, ref, rtol=1e-2, atol=1e-2)
    # and against the two-kernel path (which rounds d(act) to bf16 in between)
    two = F.swiglu_bwd(F.gemm(dout.to(DEV), w_out.to(DEV), trans_b=True), gv.to(DEV))
    close(out, two, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("B,T,heads,D,K", [(1, 256, 2, 128, 64), (3, 200, 3, 128, 136), (2, 1024, 16, 128, 256),
                                           (4, 96, 5, 64, 72), (2, 512, 12, 64, 264), (20, 512, 4, 128, 128)])
def test_gemm_with_delta_epilogue(B, T, heads, D, K):
    """dO = dY W_O^T and delta[b, h, t] = sum_d dO * O from one GEMM (ragged M and N, both head widths, a
    last round of half tiles for the largest case)."""
    M, N = B * T, heads * D
    dy = bf(M, K, seed=51)
    w_o = bf(N, K, scale=0.3, seed=52)
    o = bf(M, N, seed=53)
    assert F.gemm_delta_fusable(dy.to(DEV), w_o.to(DEV), o.to(DEV), T, D)
    do_ref = dy.float() @ w_o.float().t()
    do, delta = F.gemm_delta(dy.to(DEV), w_o.to(DEV), o.to(DEV), T, D)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    close(do, do_ref, rtol=1e-2, atol=1e-2)
    assert torch.equal(do, F.gemm(dy.to(DEV), w_o.to(DEV), trans_b=True))      # same bits as the plain GEMM
    # delta from dO as stored (bf16), like the stand-alone kernel
    ref = (do.float().cpu().view(B, T, heads, D) * o.float().view(B, T, heads, D)).sum(-1).permute(0, 2, 1)
    assert delta.shape == (B, heads, T)
    close(delta, ref, rtol=2e-3, atol=2e-3, frob=1e-3)


@pytest.mark.parametrize("M,V,K", [(256, 256, 64), (300, 1000, 136), (1024, 4096, 256), (520, 2000, 72)])
def test_lm_head_gemms_with_loss_epilogues(M, V, K):
    """Forward: logits never stored, per-tile row statistics merged into the row's log-sum-exp and the target's
    logit. Backward: (softmax - onehot) * coef formed on the recomputed accumulator, chunk by chunk."""
    x = bf(M, K, seed=31)
    w = bf(V, K, scale=0.5, seed=32)
    g = torch.Generator().manual_seed(33)
    t = torch.randint(0, V, (M,), generator=g, dtype=torch.int32)
    t[::7] = 0                                        # pad id: no loss, no gradient
    t[3] = V - 1
    logits = x.float() @ w.float().t()
    xd, wd, td = x.to(DEV), w.to(DEV), t.to(DEV)
    assert F.gemm_ce_fusable(xd, wd)
    tlogit = torch.zeros(M, device=DEV)
    pmax, psum = F.gemm_ce_stats(xd, wd, td, tlogit)
    rmax, rsum = F.ce_merge(pmax, psum)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    lse_ref = torch.logsumexp(logits, -1)
    close(rmax + torch.log(rsum), lse_ref, rtol=1e-3, atol=2e-2)
    close(tlogit, logits[torch.arange(M), t.long()], rtol=1e-3, atol=2e-2)
    loss_cnt = F.ce_loss(rmax, rsum, tlogit, td, 0)
    valid = t != 0
    ref_loss = (lse_ref - logits[torch.arange(M), t.long()])[valid].sum()
    assert abs(loss_cnt[0].item() - ref_loss.item()) <= 2e-3 * abs(ref_loss.item()) + 1e-2
    assert loss_cnt[1].item() == float(valid.sum())
    gscale = 3.0
    lse, coef = F.ce_row_coef(rmax, rsum, td, loss_cnt, 0, gscale)
    p = torch.softmax(logits, -1)
    p[torch.arange(M), t.long()] -= 1.0
    ref = p * (valid.float() * gscale / valid.sum())[:, None]
    chunk = 512 if V > 512 else V
    for s0 in range(0, V, chunk):
        e0 = min(s0 + chunk, V)
        if (e0 - s0) % 8 or e0 - s0 < 256:
            continue
        d = F.gemm_ce_dlogits(xd, wd[s0:e0], td, lse, coef, col0=s0)
        torch.cuda.synchronize()
        assert F.native.read_status() == (0, 0)
        close(d, ref[:, s0:e0], rtol=2e-2, atol=1e-6, frob=2e-2)


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_accumulate_and_fp32(bn):
    a, b = bf(300, 264, seed=3), bf(264, 520, seed=4)
    c = torch.randn(300, 520)
    ref = a.float() @ b.float() * 0.5 + c
    out = F.gemm(a.to(DEV), b.to(DEV), add=c.to(DEV), out_dtype=torch.float32, alpha=0.5, bn=bn)
    close(out, ref, rtol=1e-5, atol=1e-3)
    # accumulate in place, bf16
    acc = c.to(torch.bfloat16).to(DEV)
    F.gemm(a.to(DEV), b.to(DEV), out=acc, add=acc, bn=bn)
    close(acc, a.float() @ b.float() + c.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


def test_gemm_canary_bounds():
    """Output rows/cols outside the logical matrix must stay untouched (ragged tile edges)."""
    M, N, K = 130, 264, 72
    a, b = bf(M, K, seed=5).to(DEV), bf(K, N, seed=6).to(DEV)
    big = torch.full((M + 2, N + 16), 7.0, dtype=torch.bfloat16, device=DEV)
    view = big[1:M + 1, 8:8 + N]
    F.gemm(a, b, out=view)
    torch.cuda.synchronize()
    assert (big[0] == 7).all() and (big[-1] == 7).all()
    assert (big[:, :8] == 7).all() and (big[:, 8 + N:] == 7).all()
    close(view, a.float().cpu() @ b.float().cpu(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,H", [(37, 128), (512, 2048), (64, 4096), (9, 100), (1203, 2048), (67, 1536), (10, 8192),
                                 (3001, 3072)])
def test_rmsnorm(M, H):
    x, g, dy, res = bf(M, H, seed=1), bf(H, seed=2) * 0.1 + 1, bf(M, H, seed=3), bf(M, H, seed=4)
    y_ref, r_ref = F.rmsnorm_fwd(x.float(), g.float())
    y, r = F.rmsnorm_fwd(x.to(DEV), g.to(DEV))
    close(y, y_ref)
    close(r, r_ref, rtol=1e-4, atol=1e-5)
    dx_ref, dg_ref = F.rmsnorm_bwd(dy.float(), x.float(), g.float(), r_ref, add=res.float())
    dx, dg = F.rmsnorm_bwd(dy.to(DEV), x.to(DEV), g.to(DEV), r, add=res.to(DEV))
    close(dx, dx_ref)
    close(dg, dg_ref, rtol=2e-2, atol=5e-2)


@pytest.mark.parametrize("M,I", [(33, 512), (256, 5504), (7, 37)])
def test_swiglu(M, I):
    gv, d = bf(M, 2 * I, seed=1), bf(M, I, seed=2)
    close(F.swiglu_fwd(gv.to(DEV)), F.swiglu_fwd(gv.float()))
    close(F.swiglu_bwd(d.to(DEV), gv.to(DEV)), F.swiglu_bwd(d.float(), gv.float()))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [8 * 1000, 12345, 5])
def test_dropout_with_packed_mask_matches_the_cpu_restatement(dt, n):
    """Same (seed, offset) -> bit-identical mask on CPU and GPU; forward and backward apply it."""
    x = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(dt)
    out_c, mask_c = F.dropout_fwd(x, 0.3, 987654321, 4096)
    out_g, mask_g = F.dropout_fwd(x.to(DEV), 0.3, 987654321, 4096)
    torch.cuda.synchronize()
    assert mask_g.numel() == (n + 7) // 8 and torch.equal(mask_g.cpu(), mask_c)
    close(out_g, out_c.float(), rtol=1e-2, atol=1e-6, frob=1e-2)
    g = torch.randn(n, generator=torch.Generator().manual_seed(1)).to(dt)
    close(F.dropout_bwd(g.to(DEV), mask_g, 0.3), F.dropout_bwd(g, mask_c, 0.3).float(), rtol=1e-2, atol=1e-6)
    assert F.native.read_status() == (0, 0)


def test_rope_roundtrip_and_reference():
    T, D, H = 64, 32, 6
    buf = bf(2 * T, 8 + H * D, seed=1)
    cos_c, sin_c = F.rope_table(T, D, 10000.0, "cpu")
    cos_g, sin_g = F.rope_table(T, D, 10000.0, DEV)
    close(cos_g, cos_c, rtol=1e-4, atol=1e-4)
    ref = F.rope_inplace(buf.float().clone(), cos_c, sin_c, T, H, D, col0=8)
    out = F.rope_inplace(buf.to(DEV).clone(), cos_g, sin_g, T, H, D, col0=8)
    close(out, ref)
    back = F.rope_inplace(out.clone(), cos_g, sin_g, T, H, D, col0=8, inverse=True)
    close(back, buf, rtol=3e-2, atol=3e-2)


def test_embedding():
    V, H, M, pad = 97, 64, 300, 2
    W = bf(V, H, seed=1)
    idx = torch.randint(0, V, (M,), dtype=torch.int32)
    out = F.embedding_fwd(W.to(DEV), idx.to(DEV), pad)
    close(out, F.embedding_fwd(W.float(), idx, pad), rtol=0, atol=0)
    dout = bf(M, H, seed=2)
    for dt in (torch.float32, torch.bfloat16):
        dW = torch.zeros(V, H, dtype=dt, device=DEV)
        F.embedding_bwd(dW, idx.to(DEV), dout.to(DEV), pad)
        ref = F.embedding_bwd(torch.zeros(V, H), idx, dout.float(), pad)
        close(dW, ref, rtol=2e-2, atol=6e-2)
        assert (dW[pad] == 0).all()


def test_embedding_rejects_ids_beyond_the_vocabulary():
    """A token id >= V touches no memory: zeros forward, no update backward, status error 4."""
    V, H, M, pad = 50, 64, 40, 0
    W = bf(V, H, seed=3).to(DEV)
    idx = torch.randint(1, V, (M,), dtype=torch.int32)
    idx[7] = V          # first row past the table
    idx[19] = 1 << 20
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    out = F.embedding_fwd(W, idx.to(DEV), pad)
    assert F.native.read_status() == (4, 401)
    good = idx.clone()
    good[7] = pad
    good[19] = pad
    close(out, F.embedding_fwd(W.float().cpu(), good, pad), rtol=0, atol=0)
    dW = torch.zeros(V, H, dtype=torch.float32, device=DEV)
    dout = bf(M, H, seed=4).to(DEV)
    F.embedding_bwd(dW, idx.to(DEV), dout, pad)
    assert F.native.read_status() == (4, 402)
    close(dW, F.embedding_bwd(torch.zeros(V, H), good, dout.float().cpu(), pad), rtol=1e-5, atol=1e-5)
    assert F.native.read_status() == (0, 0)


@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("rope", [False, True])
def test_flash_attention(D, rope):
    B, T, QH, KVH = 2, 200, 4, 2
    packed = bf(B * T, (QH + 2 * KVH) * D, seed=D).to(DEV)        # [K | Q | V] columns
    v3 = packed.view(B, T, -1)
    k = v3[:, :, :KVH * D].unflatten(2, (KVH, D))
    q = v3[:, :, KVH * D:(KVH + QH) * D].unflatten(2, (QH, D))
    v = v3[:, :, (KVH + QH) * D:].unflatten(2, (KVH, D))
    vl = torch.tensor([T, 150], dtype=torch.int32, device=DEV)
    tabs = F.rope_table(T, D, 10000.0, DEV) if rope else None
    tabs_c = F.rope_table(T, D, 10000.0, "cpu") if rope else None
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vl, rope=tabs)
    qc, kc, vc = q.float().cpu(), k.float().cpu(), v.float().cpu()
    o_ref, lse_ref = F.flash_attn_fwd(qc, kc, vc, valid_len=vl.cpu(), rope=tabs_c)
    close(o, o_ref)
    close(lse, lse_ref, rtol=1e-2, atol=2e-2)
    do = bf(B, T, QH, D, seed=9).to(DEV)
    dq, dk, dv = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vl, rope=tabs)
    dq_r, dk_r, dv_r = F.flash_attn_bwd(do.float().cpu(), qc, kc, vc, o_ref, lse_ref, valid_len=vl.cpu(), rope=tabs_c)
    close(dq, dq_r, rtol=3e-2, atol=3e-2)
    close(dk, dk_r, rtol=3e-2, atol=3e-2)
    close(dv, dv_r, rtol=3e-2, atol=3e-2)


def test_decode_attention():
    B, QH, KVH, Tmax, D = 3, 8, 2, 77, 64
    q, kc, vc = bf(B, QH, D, seed=1), bf(B, KVH, Tmax, D, seed=2), bf(B, KVH, Tmax, D, seed=3)
    lens = torch.tensor([1, 40, 77], dtype=torch.int32)
    out = F.decode_attn(q.to(DEV), kc.to(DEV), vc.to(DEV), lens.to(DEV))
    close(out, F.decode_attn(q.float(), kc.float(), vc.float(), lens))


def test_cross_entropy_rows():
    M, V, C, pad = 100, 1000, 384, 2
    logits = torch.randn(M, V) * 3
    tg = torch.randint(0, V, (M,), dtype=torch.int32)
    tg[::7] = pad
    dev = lambda t: t.to(DEV)
    st_g = [torch.empty(M, device=DEV) for _ in range(3)]
    st_c = [torch.empty(M) for _ in range(3)]
    for i, c0 in enumerate(range(0, V, C)):
        ch = logits[:, c0:c0 + C].contiguous()
        F.ce_stats(dev(ch), dev(tg), *st_g, c0, i == 0)
        F.ce_stats(ch, tg, *st_c, c0, i == 0)
    lc_g = F.ce_loss(*st_g, dev(tg), pad)
    lc_c = F.ce_loss(*st_c, tg, pad)
    close(lc_g, lc_c, rtol=1e-4, atol=1e-3)
    ref = torch.nn.functional.cross_entropy(logits, tg.long(), ignore_index=pad, reduction="sum")
    assert abs(lc_g[0].item() - ref.item()) < 1e-2 * abs(ref.item())
    ch = logits[:, C:2 * C].contiguous()
    d_g = F.ce_dlogits(dev(ch), dev(tg), st_g[0], st_g[1], lc_g, C, pad, 4.0, torch.bfloat16)
    d_c = F.ce_dlogits(ch, tg, st_c[0], st_c[1], lc_c, C, pad, 4.0, torch.float32)
    close(d_g, d_c, rtol=2e-2, atol=1e-4)


@pytest.mark.parametrize("gdt", [torch.bfloat16, torch.float32])
def test_adamw_and_stats(gdt):
    n = 10007
    g = torch.randn(n).to(gdt)
    w = torch.randn(n)
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-6, weight_decay=0.1)
    st_c = torch.zeros(2)
    F.grad_stats(g.float(), st_c)
    st_g = torch.zeros(2, device=DEV)
    F.grad_stats(g.to(DEV), st_g)
    close(st_g, st_c, rtol=1e-3, atol=1e-3)
    mc, vc, wc, pc = torch.zeros(n), torch.zeros(n), w.clone(), torch.zeros(n)
    mg, vg, wg = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV), w.to(DEV)
    pg = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    for step in (1, 2, 3):
        F.adamw_step(g.float(), mc, vc, wc, pc, step=step, grad_scale=0.5, max_grad_norm=1.0, stats=st_c, **hp)
        F.adamw_step(g.to(DEV), mg, vg, wg, pg, step=step, grad_scale=0.5, max_grad_norm=1.0, stats=st_g, **hp)
    close(wg, wc, rtol=1e-4, atol=1e-5)
    close(pg, pc, rtol=1e-2, atol=1e-2)
    # non-finite gradient: flagged, and the update is skipped on the device
    gb = g.clone().float()
    gb[5] = float("inf")
    st = torch.zeros(2, device=DEV)
    F.grad_stats(gb.to(gdt).to(DEV), st)
    assert st[1].item() == 1.0
    before = wg.clone()
    F.adamw_step(gb.to(gdt).to(DEV), mg, vg, wg, pg, step=4, stats=st, **hp)
    assert torch.equal(before, wg)
    acc = torch.zeros(n, device=DEV)
    F.accumulate(acc, g.to(DEV), 0.25)
    close(acc, g.float() * 0.25, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("off,n", [(0, 100_003), (1, 77_777), (3, 5), (5, 1 << 20), (2, 4099)])
def test_grad_stats_unaligned_slices(dt, off, n):
    """The vector body starts at the first 16-byte boundary; head and tail are read one by one."""
    g = (torch.randn(n + 16, generator=torch.Generator().manual_seed(n)) * 3).to(dt)
    ref = float((g[off:off + n].float() ** 2).sum())
    st = torch.zeros(2, device=DEV)
    F.grad_stats(g.to(DEV)[off:off + n], st)
    assert abs(st[0].item() - ref) <= 2e-3 * ref and st[1].item() == 0.0
    gb = g.clone()
    gb[off + n - 1] = float("nan")
    st.zero_()
    F.grad_stats(gb.to(DEV)[off:off + n], st)
    assert st[1].item() == 1.0
    gb = g.clone()
    gb[off] = float("inf")
    st.zero_()
    F.grad_stats(gb.to(DEV)[off:off + n], st)
    assert st[1].item() == 1.0


@pytest.mark.parametrize("T,vl", [(640, None), (333, [333, 100])])
def test_flash_attention_tcgen05_multi_tile(T, vl):
    """head_dim 128 without in-kernel RoPE runs the tcgen05/TMEM kernels (forward, dQ, dK/dV)."""
    B, QH, KVH, D = 2, 8, 2, 128
    g = torch.Generator().manual_seed(T)
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    do = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    vlt = None if vl is None else torch.tensor(vl, dtype=torch.int32, device=DEV)
    assert F.FLASH_TC and F.FLASH_TC_BWD
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vlt)
    dq, dk, dv = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    qc, kc, vc = q.float().cpu(), k.float().cpu(), v.float().cpu()
    vlc = None if vlt is None else vlt.cpu()
    o_r, lse_r = F.flash_attn_fwd(qc, kc, vc, valid_len=vlc)
    r = F.flash_attn_bwd(do.float().cpu(), qc, kc, vc, o_r, lse_r, valid_len=vlc)
    close(o, o_r)
    close(lse, lse_r, rtol=1e-2, atol=2e-2)
    for a, b in zip((dq, dk, dv), r):
        close(a, b, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("B,T,QH,KVH,vl", [(1, 256, 2, 1, None), (2, 520, 4, 2, [520, 300]), (2, 1024, 8, 2, None),
                                          (3, 384, 4, 4, [384, 129, 1])])
def test_flash_backward_both_dkv_schedules_match_the_reference(B, T, QH, KVH, vl):
    """head_dim 128: the dK/dV kernel with 128-query iterations (default) and the one with double-buffered
    64-query iterations against the fp32 restatement, with ragged lengths and a padded tail."""
    D = 128
    q, k, v, do = (bf(B, T, h, D, seed=60 + i).to(DEV) for i, h in enumerate((QH, KVH, KVH, QH)))
    valid = None if vl is None else torch.tensor(vl, dtype=torch.int32, device=DEV)
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=valid)
    qc, kc, vc = q.float().cpu(), k.float().cpu(), v.float().cpu()
    vlc = None if valid is None else valid.cpu()
    o_r, lse_r = F.flash_attn_fwd(qc, kc, vc, valid_len=vlc)
    ref = F.flash_attn_bwd(do.float().cpu(), qc, kc, vc, o_r, lse_r, valid_len=vlc)
    assert F.flash_bwd_wide_active()       # on a B200 the 128-query kernel is what runs, not its fallback
    try:
        for wide in (True, False):
            for pairing in (0, 1):       # one key tile per CTA, or tiles i and n - 1 - i (the training step's schedule)
                F.set_flash_bwd_wide(wide)
                F.set_flash_bwd_pairing(pairing)
                got = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=valid)
                torch.cuda.synchronize()
                assert F.native.read_status() == (0, 0)
                for a, b in zip(got, ref):
                    close(a, b, rtol=3e-2, atol=3e-2, frob=2e-2)
    finally:
        F.set_flash_bwd_wide(True)
        F.set_flash_bwd_pairing(-1)


def test_flash_backward_unpaired_key_tile_schedule():
    """With at least three key tiles per SM in flight (here 8 x 8 x 8 = 512 on 148 SMs) a dK/dV CTA owns ONE key
    tile, longest first; between one and three per SM a CTA owns tiles i and n - 1 - i (the 1.3 B training step)."""
    B, T, QH, KVH, D = 8, 1024, 8, 8, 128
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    do = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    vlt = torch.tensor([T, T, 700, T, 1, T, 513, T], dtype=torch.int32, device=DEV)
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vlt)
    dq, dk, dv = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    o_r, lse_r = F.flash_attn_fwd(q.float().cpu(), k.float().cpu(), v.float().cpu(), valid_len=vlt.cpu())
    r = F.flash_attn_bwd(do.float().cpu(), q.float().cpu(), k.float().cpu(), v.float().cpu(), o_r, lse_r,
                         valid_len=vlt.cpu())
    close(o, o_r)
    for a, b in zip((dq, dk, dv), r):
        close(a, b, rtol=3e-2, atol=3e-2, frob=1.5e-2)


def test_kernels_without_atomics_are_bitwise_reproducible():
    """Run-to-run comparison in place of a race detector: the GEMM (both tile schedulers), the attention
    forward and the attention backward have no atomics and no order-dependent reductions, so two launches
    on the same inputs must agree bit for bit; a data race between warps or CTAs would show up here."""
    g = torch.Generator().manual_seed(11)
    a = torch.randn(1024, 512, generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randn(512, 1536, generator=g).to(torch.bfloat16).to(DEV)
    outs = [F.gemm(a, b) for _ in range(3)] + [F.gemm(a, b, impl="1cta")]
    assert all(torch.equal(outs[0], o) for o in outs[1:3])
    B, T, QH, KVH, D = 2, 640, 8, 2, 128
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    do = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    runs = []
    for _ in range(2):
        o, lse = F.flash_attn_fwd(q, k, v)
        runs.append((o, lse) + tuple(F.flash_attn_bwd(do, q, k, v, o, lse)))
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    for x, y in zip(*runs):
        assert torch.equal(x, y)


@pytest.mark.parametrize("T,vl", [(128, None), (333, [333, 100]), (640, [640, 300]), (1000, None)])
def test_flash_head_dim_64_on_tcgen05(T, vl, monkeypatch):
    """head_dim 64 runs the same tcgen05 forward and backward kernels (template parameter); checked against
    fp32 and against the mma.sync kernels they replace."""
    B, QH, KVH, D = 2, 6, 2, 64
    g = torch.Generator().manual_seed(T + 64)
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    vlt = None if vl is None else torch.tensor(vl, dtype=torch.int32, device=DEV)
    assert F.flash_tc_forward_dim(D)
    n0 = F.native.launch_count()
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vlt)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0) and F.native.launch_count() == n0 + 1
    o_r, lse_r = F.flash_attn_fwd(q.float().cpu(), k.float().cpu(), v.float().cpu(),
                                  valid_len=None if vlt is None else vlt.cpu())
    close(o, o_r)
    ok = torch.isfinite(lse_r)
    close(lse.cpu()[ok], lse_r[ok], rtol=1e-2, atol=2e-2)
    do = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    n0 = F.native.launch_count()
    dq, dk, dv = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt)     # delta, dK/dV (+ dS^T), dQ GEMM
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0) and F.native.launch_count() == n0 + 3
    r = F.flash_attn_bwd(do.float().cpu(), q.float().cpu(), k.float().cpu(), v.float().cpu(), o_r, lse_r,
                         valid_len=None if vlt is None else vlt.cpu())
    for a, b in zip((dq, dk, dv), r):
        close(a, b, rtol=3e-2, atol=3e-2)
    monkeypatch.setattr(F, "FLASH_TC_D64", False)          # the mma.sync kernels this path replaces
    o2, lse2 = F.flash_attn_fwd(q, k, v, valid_len=vlt)
    close(o, o2)
    for a, b in zip((dq, dk, dv), F.flash_attn_bwd(do, q, k, v, o2, lse2, valid_len=vlt)):
        close(a, b, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("D", [64, 128])
def test_flash_backward_in_batch_chunks(D, monkeypatch):
    """When the dS^T workspace of the whole batch exceeds the limit, the backward runs chunk by chunk."""
    B, T, QH, KVH = 3, 300, 4, 2
    g = torch.Generator().manual_seed(D)
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    do = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    vlt = torch.tensor([300, 17, 200], dtype=torch.int32, device=DEV)
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vlt)
    whole = [t.clone() for t in F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt)]
    monkeypatch.setattr(F, "FLASH_DQ_GEMM_MAX_BYTES", QH * 384 * 384 * 2)        # room for one batch element
    assert F._ds_batch_chunk(B, QH, T) == 1
    n0 = F.native.launch_count()
    parts = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0) and F.native.launch_count() == n0 + 1 + 2 * B
    for a, b in zip(parts, whole):
        assert torch.equal(a, b)
    # not even one batch element fits: one KV-head group (QH / KVH query heads) of one batch element per call
    monkeypatch.setattr(F, "FLASH_DQ_GEMM_MAX_BYTES", (QH // KVH) * 384 * 384 * 2)
    assert F._ds_batch_chunk(B, QH, T) == 0
    n0 = F.native.launch_count()
    parts = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0) and F.native.launch_count() == n0 + 1 + 2 * B * KVH
    for a, b in zip(parts, whole):
        assert torch.equal(a, b)


@pytest.mark.parametrize("D,dq_gemm", [(128, True), (128, False), (64, True)])
@pytest.mark.parametrize("T,vl", [(640, None), (333, [333, 100])])
def test_flash_backward_unrotates_in_the_epilogue(T, vl, D, dq_gemm, monkeypatch):
    """unrotate=(cos, sin): dQ and dK leave the tcgen05 backward kernels with the inverse rotary embedding
    applied (both dQ kernels and the dK/dV kernel), equal to the fp32 restatement."""
    monkeypatch.setattr(F, "FLASH_DQ_GEMM", dq_gemm)
    monkeypatch.setattr(F, "FLASH_ROPE_EPILOGUE_D64", True)
    B, QH, KVH = 2, 8, 2
    g = torch.Generator().manual_seed(T + 1)
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    do = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    vlt = None if vl is None else torch.tensor(vl, dtype=torch.int32, device=DEV)
    tabs = F.rope_table(T + 5, D, 10000.0, DEV)
    assert F.flash_bwd_can_unrotate(q)
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vlt)
    dq, dk, dv = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt, unrotate=tabs)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    qc, kc, vc = q.float().cpu(), k.float().cpu(), v.float().cpu()
    vlc = None if vlt is None else vlt.cpu()
    o_r, lse_r = F.flash_attn_fwd(qc, kc, vc, valid_len=vlc)
    r = F.flash_attn_bwd(do.float().cpu(), qc, kc, vc, o_r, lse_r, valid_len=vlc,
                         unrotate=tuple(t.cpu() for t in tabs))
    for a, b in zip((dq, dk, dv), r):
        close(a, b, rtol=3e-2, atol=3e-2)
    # and the two-step form (kernels, then the in-place pass) agrees to bf16 rounding
    dq2, dk2, dv2 = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vlt)
    F.rope_inplace(dq2.view(B * T, QH * D), tabs[0], tabs[1], T, QH, D, inverse=True)
    F.rope_inplace(dk2.view(B * T, KVH * D), tabs[0], tabs[1], T, KVH, D, inverse=True)
    close(dq, dq2.float().cpu(), rtol=2e-2, atol=2e-2)
    close(dk, dk2.float().cpu(), rtol=2e-2, atol=2e-2)
    assert torch.equal(dv, dv2)


@pytest.mark.parametrize("T,vl", [(128, None), (384, None), (640, [640, 300]), (1000, None)])
def test_flash_forward_tile_edges(T, vl):
    """The tcgen05 forward kernel against the fp32 reference; T = 384 leaves the second query tile of the
    last pair empty, T = 1000 ends inside a tile."""
    B, QH, KVH, D = 2, 4, 2, 128
    g = torch.Generator().manual_seed(T + 3)
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    vlt = None if vl is None else torch.tensor(vl, dtype=torch.int32, device=DEV)
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vlt)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    o_r, lse_r = F.flash_attn_fwd(q.float().cpu(), k.float().cpu(), v.float().cpu(),
                                  valid_len=None if vlt is None else vlt.cpu())
    close(o, o_r)
    close(lse, lse_r, rtol=1e-2, atol=2e-2)


def test_flash_forward_moving_maximum():
    """Keys whose norm grows along the sequence push the row maximum up tile after tile, which makes
    the kernel rescale its TMEM output accumulator."""
    B, T, QH, KVH, D = 1, 512, 2, 1, 128
    g = torch.Generator().manual_seed(1)
    q = (torch.randn(B, T, QH, D, generator=g) * 3).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, T, KVH, D, generator=g) * torch.linspace(0.2, 4.0, T)[None, :, None, None]
    k = k.to(torch.bfloat16).to(DEV)
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).to(DEV)
    o, lse = F.flash_attn_fwd(q, k, v)
    torch.cuda.synchronize()
    assert F.native.read_status() == (0, 0)
    o_r, lse_r = F.flash_attn_fwd(q.float().cpu(), k.float().cpu(), v.float().cpu())
    close(o, o_r, rtol=3e-2, atol=3e-2)
    close(lse, lse_r, rtol=1e-3, atol=1e-2)


def test_bounds_checking_build_reports_out_of_range_device_arguments():
    """The debug library (-DB200_BOUNDS_CHECK=1): a valid length beyond the sequence and a target id beyond the
    vocabulary are reported through the status word (error 4, kernel id, the value) and clamped; in-range
    arguments leave the status clear. The regular library clamps silently."""
    import json
    import os
    import subprocess
    import sys

    script = os.path.join(os.path.dirname(__file__), "bounds_check_child.py")
    res = {}
    for flag in ("1", "0"):
        env = dict(os.environ, B200_BOUNDS_CHECK=flag)
        r = subprocess.run([sys.executable, script], env=env, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        res[flag] = json.loads(r.stdout.strip().splitlines()[-1])
    dbg, rel = res["1"], res["0"]
    assert dbg["lib"] == "libb200llm_dbg.so" and dbg["bounds_check"] and rel["lib"] == "libb200llm.so"
    assert dbg["in_range"] == [0, 0] and dbg["targets_in_range"] == [0, 0]
    assert dbg["too_long"] == [4, 301, 256 + 5] and dbg["clamped_equal"]
    assert dbg["target_beyond_vocab"] == [4, 304, 512 + 3]
    assert rel["too_long"][0] == 0 and rel["target_beyond_vocab"][0] == 0 and rel["clamped_equal"]
