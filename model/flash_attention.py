"""``model.flash_attention`` of the reference, with the reference's call signatures
(model/flash_attention.py:51, :109, :252): tensors in the grouped layout ``Q [B, KVH, R, T, D]``,
``K / V [B, KVH, T, D]``, ``O [B, KVH, R, T, D]``, ``LSE [B, KVH, R, T]``; Q and K are expected rotated
already and ``scale`` is applied inside, as there. The work is done by the native causal GQA kernels,
which take ``[B, T, heads, D]`` views with arbitrary strides, so the adapters only permute views; the
tile-size arguments of the reference are accepted and ignored (the kernels choose their own tiles).
"""
from create_llm_by_cupy_b200.ops.functional import decode_attn, flash_attn_bwd, flash_attn_fwd  # noqa: F401
from create_llm_by_cupy_b200.utils.functions import pad_mask_to_valid_len


def _to_bthd(Q, K, V):
    B, KVH, R, T, D = Q.shape
    q = Q.permute(0, 3, 1, 2, 4).reshape(B, T, KVH * R, D)      # head index h = kvh * R + r, as in the reference
    k = K.permute(0, 2, 1, 3)
    v = V.permute(0, 2, 1, 3)
    return q, k, v


def _valid_len(pad_mask, T):
    return None if pad_mask is None else pad_mask_to_valid_len(pad_mask, T)


def cupy_flash_gqa_forward(Q, K, V, pad_mask, scale, block_m=64, block_n=64):
    """Exact causal GQA attention forward. Returns ``(O [B, KVH, R, T, D], LSE [B, KVH, R, T] fp32)``.
    ``pad_mask``: additive key mask (e.g. ``[B, 1, 1, T]``), boolean mask or valid lengths, or None."""
    B, KVH, R, T, D = Q.shape
    q, k, v = _to_bthd(Q, K, V)
    o, lse = flash_attn_fwd(q, k, v, valid_len=_valid_len(pad_mask, T), scale=float(scale), rope=None)
    return o.view(B, T, KVH, R, D).permute(0, 2, 3, 1, 4), lse.view(B, KVH, R, T)


def cupy_flash_gqa_backward(Q, K, V, dO, O, LSE, pad_mask, scale, block_m=32, block_n=64):
    """Exact causal GQA attention backward. Returns ``(dQ [B, KVH, R, T, D], dK, dV [B, KVH, T, D])``."""
    B, KVH, R, T, D = Q.shape
    q, k, v = _to_bthd(Q, K, V)
    do = dO.permute(0, 3, 1, 2, 4).reshape(B, T, KVH * R, D)
    o = O.permute(0, 3, 1, 2, 4).reshape(B, T, KVH * R, D)
    dq, dk, dv = flash_attn_bwd(do, q, k, v, o, LSE.reshape(B, KVH * R, T), valid_len=_valid_len(pad_mask, T),
                                scale=float(scale), rope=None)
    return (dq.view(B, T, KVH, R, D).permute(0, 2, 3, 1, 4), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3))


def triton_flash_gqa_forward(Q, K, V, valid_lens, scale, block_m=64, block_n=64, block_d=None):
    """The reference's optional Triton forward (valid lengths instead of a mask): the same native kernel."""
    return cupy_flash_gqa_forward(Q, K, V, valid_lens, scale)


def triton_is_available() -> bool:
    """There is no Triton path in this stack; the native kernels are always the backend."""
    return False
