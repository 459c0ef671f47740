"""Tiny-config model on the CPU path against the NumPy float64 oracle (loss, every gradient,
Adam steps, greedy decode), plus a finite-difference check of the oracle itself."""
import numpy as np
import pytest
import torch

from create_llm_by_cupy_b200.models.model import Cupa_ver4
from create_llm_by_cupy_b200.models.oracle_np import Oracle, OracleConfig

TINY = dict(vocab_size=64, hidden_size=32, layer_num=2, time_size=16, q_head=4, kv_head=2, padding_id=2,
            dropout_rate=0, half_float=False, dtype="fp32", ffn_size=48, tie_embeddings=True, seed=3,
            ce_chunk_size=24)


def make(tied=True, **kw):
    d = dict(TINY, tie_embeddings=tied, **kw)
    m = Cupa_ver4(d, device="cpu")
    o = Oracle(OracleConfig.from_model_dic(d), [p.double().numpy() for p in m.params])
    return d, m, o


def batch(d, B=3, seed=0, pad_tail=True):
    rng = np.random.default_rng(seed)
    x = rng.integers(3, d["vocab_size"], size=(B, d["time_size"]))
    t = np.concatenate([x[:, 1:], np.full((B, 1), d["padding_id"])], 1)
    vl = np.full(B, d["time_size"])
    if pad_tail:
        vl[1] = 11
        x[1, 10:] = d["padding_id"]
        t[1, 10:] = d["padding_id"]
    return x, t, vl


def test_oracle_gradients_match_finite_differences():
    d, m, o = make()
    x, t, vl = batch(d)
    o.forward(x, t, vl)
    grads = o.backward()
    rng = np.random.default_rng(1)
    for pi in (0, 1, 2, 3, 4, 6, 12, len(o.p) - 1):
        p = o.p[pi]
        for _ in range(3):
            idx = tuple(rng.integers(0, s) for s in p.shape)
            old = p[idx]
            h = 1e-5
            p[idx] = old + h
            lp = o.forward(x, t, vl, keep=False)
            p[idx] = old - h
            lm = o.forward(x, t, vl, keep=False)
            p[idx] = old
            fd = (lp - lm) / (2 * h)
            assert abs(fd - grads[pi][idx]) < 1e-6 + 1e-4 * abs(fd), (pi, idx, fd, grads[pi][idx])


@pytest.mark.parametrize("tied", [True, False])
@pytest.mark.parametrize("flash", ["b200", "none"])
def test_torch_cpu_matches_oracle(tied, flash):
    d, m, o = make(tied, flash_backend=flash)
    x, t, vl = batch(d)
    loss = m.forward(torch.from_numpy(x), torch.from_numpy(t), torch.from_numpy(vl).int())
    ref = o.forward(x, t, vl)
    assert abs(float(loss) - ref) < 1e-4
    m.backward(GradScale=2.0)
    g_ref = o.backward(2.0)
    assert len(m.grads) == len(g_ref)
    for i, (g, r) in enumerate(zip(m.grads, g_ref)):
        np.testing.assert_allclose(g.double().numpy(), r, rtol=2e-3, atol=2e-5, err_msg=f"param {i}")


def test_recompute_switches_give_same_gradients():
    d, m, _ = make()
    x, t, vl = batch(d)
    X, Tt, V = torch.from_numpy(x), torch.from_numpy(t), torch.from_numpy(vl).int()
    m.forward(X, Tt, V)
    m.backward()
    base = [g.clone() for g in m.grads]
    m2 = Cupa_ver4(dict(d, gqa_cache_out_value=False, gqa_cache_kqv=False, swiglu_cache_gate=False,
                        ce_cache_logits=False, keep_layer_num=2), device="cpu")
    m2.forward(X, Tt, V)
    m2.backward()
    for a, b in zip(base, m2.grads):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_predict_and_logits_and_greedy_generation():
    d, m, o = make()
    x, t, vl = batch(d, pad_tail=False)
    lp = m.predict(torch.from_numpy(x), torch.from_numpy(t), None)
    assert abs(float(lp) - o.forward(x, t, None, keep=False)) < 1e-4
    lg = m.logits(torch.from_numpy(x))
    np.testing.assert_allclose(lg.double().numpy(), o.logits(x), rtol=1e-3, atol=1e-4)
    prompt = [5, 9, 33, 7]
    out = m.generate(prompt, greedy=True, max_new_tokens=8)
    assert out == o.greedy(prompt, 8)
    out2 = m.generate(prompt, start_id=1, end_id=0, temp=0.7, top=0.9, penalty=1.2, seed=0)
    assert all(0 <= tok < d["vocab_size"] and tok != d["padding_id"] for tok in out2)
    out3 = m.chat_generate(prompt, user_id=4, bot_id=6, end_id=0, seed=0, max_new_tokens=4)
    assert len(out3) <= 4


def test_flat_weight_file_roundtrip(tmp_path):
    d, m, _ = make()
    p = tmp_path / "flat_params_f16.pkl.gz"
    m.save_weights_to_flat_file(str(p))
    m2 = Cupa_ver4(dict(d, seed=99), param_path=str(p), device="cpu")
    for a, b in zip(m.params, m2.params):
        torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-3)
    assert m2.layers[0].params[0] is m2.params[0]


def test_dropout_branches_and_mask_adapters():
    from create_llm_by_cupy_b200.utils.functions import pad_mask_to_valid_len
    d = dict(TINY, dropout_rate=0.25)
    m = Cupa_ver4(d, device="cpu")
    x, t, vl = batch(d)
    X, Tt, V = torch.from_numpy(x), torch.from_numpy(t), torch.from_numpy(vl).int()
    l1 = float(m.forward(X, Tt, V))
    m.backward()
    assert all(torch.isfinite(g).all() for g in m.grads)
    l_eval = float(m.predict(X, Tt, V))            # no dropout at inference
    m0 = Cupa_ver4(dict(TINY), device="cpu")
    assert abs(l_eval - float(m0.predict(X, Tt, V))) < 1e-5 and abs(l1 - l_eval) > 1e-6
    # pad-mask forms -> valid lengths
    lens = torch.tensor([16, 11, 5], dtype=torch.int32)
    add4 = m.make_mask(lens)
    assert torch.equal(pad_mask_to_valid_len(add4, 16), lens)
    assert torch.equal(pad_mask_to_valid_len(torch.isinf(add4[:, 0, 0, :]), 16), lens)
    assert torch.equal(pad_mask_to_valid_len(lens, 16), lens)
    with pytest.raises(ValueError):
        pad_mask_to_valid_len(torch.tensor([[False, True, False, False]]), 4)


def test_dropout_mask_is_bit_packed_and_attention_dropout_backward_matches_autograd():
    from create_llm_by_cupy_b200.models.layers import TimeDropout
    from create_llm_by_cupy_b200.ops import functional as F

    gen = torch.Generator().manual_seed(3)
    drop = TimeDropout(0.3, torch.float32, gen)
    x = torch.randn(5, 7, 11, generator=gen)
    y = drop.forward(x, True)
    assert drop.mask.dtype == torch.uint8 and drop.mask.numel() == (x.numel() + 7) // 8     # one bit per element
    keep = F._unpackbits(drop.mask, x.numel()).view(x.shape)
    torch.testing.assert_close(y, x * keep / 0.7)
    assert 0.55 < keep.float().mean() < 0.85
    g = torch.randn(x.shape, generator=gen)
    torch.testing.assert_close(drop.backward(g), g * keep / 0.7)
    assert drop.mask is None
    y2 = drop.forward(x, True)                         # the next call draws another mask
    assert not torch.equal(y2 != 0, y != 0)
    assert drop.forward(x, False) is x                 # inference: identity

    # attention with dropout on the probabilities: manual backward against autograd with the same mask
    B, T, QH, KVH, D = 2, 12, 4, 2, 8
    q = torch.randn(B, T, QH, D, generator=gen, requires_grad=True)
    k = torch.randn(B, T, KVH, D, generator=gen, requires_grad=True)
    v = torch.randn(B, T, KVH, D, generator=gen, requires_grad=True)
    do = torch.randn(B, T, QH, D, generator=gen)
    cos, sin = F.rope_table(T, D, 10000.0, "cpu")
    vl = torch.tensor([12, 9], dtype=torch.int32)
    scale = D ** -0.5
    adrop = TimeDropout(0.25, torch.float32, gen)
    _, _, p, _, _ = F._attn_reference(q, k, v, vl, scale, cos, sin)
    p_used = adrop.forward(p.detach(), True)
    keep = F._unpackbits(adrop.mask, p.numel()).view(p.shape)
    o = torch.einsum("bhts,bshd->bthd", p * keep / 0.75, v.repeat_interleave(QH // KVH, dim=2))
    torch.testing.assert_close(o, torch.einsum("bhts,bshd->bthd", p_used, v.detach().repeat_interleave(QH // KVH, dim=2)))
    (o * do).sum().backward()
    dq, dk, dv = F._attn_bwd_reference(do, q.detach(), k.detach(), v.detach(), o.detach(), vl, scale, cos, sin,
                                       p_drop=adrop)
    torch.testing.assert_close(dq, q.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dk, k.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dv, v.grad, rtol=1e-4, atol=1e-5)


def test_attention_backward_unrotate_equals_in_kernel_rope():
    """Two ways to the same gradients: (a) q, k un-rotated and ``rope=`` (rotation inside), (b) q, k rotated
    beforehand and ``unrotate=`` (inverse rotation of dq, dk on the way out) - the contract of the epilogue
    form on the GPU, checked here on the fp32 restatement; and the chunk sizes of the dS^T workspace."""
    import torch
    from create_llm_by_cupy_b200.ops import functional as F
    B, T, QH, KVH, D = 2, 24, 4, 2, 16
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(B, T, h, D, generator=g) for h in (QH, KVH, KVH))
    do = torch.randn(B, T, QH, D, generator=g)
    vl = torch.tensor([24, 9], dtype=torch.int32)
    tabs = F.rope_table(T, D, 10000.0, "cpu")
    o, lse = F.flash_attn_fwd(q, k, v, valid_len=vl, rope=tabs)
    ref = F.flash_attn_bwd(do, q, k, v, o, lse, valid_len=vl, rope=tabs)
    packed = torch.cat([k.reshape(B * T, -1), q.reshape(B * T, -1)], 1).clone()
    F.rope_inplace(packed, tabs[0], tabs[1], T, KVH + QH, D)
    kr = packed[:, :KVH * D].reshape(B, T, KVH, D)
    qr = packed[:, KVH * D:].reshape(B, T, QH, D)
    o2, lse2 = F.flash_attn_fwd(qr, kr, v, valid_len=vl)
    torch.testing.assert_close(o2, o, rtol=1e-5, atol=1e-5)
    got = F.flash_attn_bwd(do, qr, kr, v, o2, lse2, valid_len=vl, unrotate=tabs)
    for a, b in zip(got, ref):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    try:
        F.flash_attn_bwd(do, q, k, v, o, lse, rope=tabs, unrotate=tabs)
        raise AssertionError("rope= and unrotate= together must be refused")
    except ValueError:
        pass
    # batch elements (or, below one, KV-head groups) per call under the workspace cap
    cap = F.FLASH_DQ_GEMM_MAX_BYTES
    assert F._ds_batch_chunk(4, 16, 2048) == 4
    assert F._ds_batch_chunk(8, 32, 4096) == cap // (32 * 4096 * 4096 * 2)
    assert F._ds_batch_chunk(8, 32, 16384) == (1 if cap >= 32 * 16384 * 16384 * 2 else 0)


def test_reference_flash_attention_signatures():
    """``model.flash_attention`` keeps the reference's grouped layout and argument order."""
    from model.flash_attention import cupy_flash_gqa_backward, cupy_flash_gqa_forward, triton_flash_gqa_forward
    from create_llm_by_cupy_b200.ops import functional as F

    g = torch.Generator().manual_seed(2)
    B, KVH, R, T, D = 2, 2, 3, 10, 8
    Q = torch.randn(B, KVH, R, T, D, generator=g)
    K = torch.randn(B, KVH, T, D, generator=g)
    V = torch.randn(B, KVH, T, D, generator=g)
    dO = torch.randn(B, KVH, R, T, D, generator=g)
    lens = torch.tensor([10, 7], dtype=torch.int32)
    pad = torch.zeros(B, 1, 1, T)
    pad[1, ..., 7:] = float("-inf")
    scale = D ** -0.5
    O, LSE = cupy_flash_gqa_forward(Q, K, V, pad, scale, block_m=4, block_n=4)
    assert O.shape == (B, KVH, R, T, D) and LSE.shape == (B, KVH, R, T)
    # dense restatement in the grouped layout
    s = torch.einsum("bgrtd,bgsd->bgrts", Q, K) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()[None, None, None] & (torch.arange(T)[None, :] < lens[:, None])[:, None, None, None, :]
    s = s.masked_fill(~mask, float("-inf"))
    torch.testing.assert_close(O, torch.einsum("bgrts,bgsd->bgrtd", torch.softmax(s, -1), V), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(LSE, torch.logsumexp(s, -1), rtol=1e-4, atol=1e-5)
    O2, _ = triton_flash_gqa_forward(Q, K, V, lens, scale)
    torch.testing.assert_close(O2, O)
    Qa, Ka, Va = (t.clone().requires_grad_() for t in (Q, K, V))
    sa = (torch.einsum("bgrtd,bgsd->bgrts", Qa, Ka) * scale).masked_fill(~mask, float("-inf"))
    (torch.einsum("bgrts,bgsd->bgrtd", torch.softmax(sa, -1), Va) * dO).sum().backward()
    dQ, dK, dV = cupy_flash_gqa_backward(Q, K, V, dO, O, LSE, pad, scale)
    torch.testing.assert_close(dQ, Qa.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dK, Ka.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dV, Va.grad, rtol=1e-4, atol=1e-5)


def test_reference_rotary_helper_signatures():
    from model.fast_layers import apply_rotary_pos_emb_inplace, precompute_freqs_cis
    from create_llm_by_cupy_b200.ops import functional as F

    cos, sin = precompute_freqs_cis(8, 6)
    assert cos.shape == (6, 4)
    x = torch.randn(2, 3, 6, 8, generator=torch.Generator().manual_seed(0))
    y = apply_rotary_pos_emb_inplace(x.clone(), cos, sin)
    # same rotation as the packed in-place kernel front end ([M, heads * D] with token-major rows)
    buf = x.permute(0, 2, 1, 3).reshape(12, 24).clone()
    F.rope_inplace(buf, cos, sin, 6, 3, 8)
    torch.testing.assert_close(y, buf.view(2, 6, 3, 8).permute(0, 2, 1, 3))
    torch.testing.assert_close(apply_rotary_pos_emb_inplace(y, cos, -sin), x, rtol=1e-5, atol=1e-6)
