"""Operator front ends used by the layers.

Every function has two bodies: CUDA tensors go to the hand-written sm_100a kernels of the native
library (bf16 storage, fp32 arithmetic); CPU tensors take a plain torch restatement of the same
math in the tensor's own dtype. The CPU body is what the NumPy-oracle comparison, the gloo
multi-process tests and the CPU smoke configuration run; it is never used for CUDA tensors.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import native
from .gemm import (gemm, gemm_ce_dlogits, gemm_ce_fusable, gemm_ce_stats, gemm_delta, gemm_delta_fusable,  # noqa: F401
                   gemm_rope, gemm_rope_fusable,
                   gemm_swiglu, gemm_swiglu_bwd, gemm_swiglu_bwd_fusable, gemm_swiglu_fusable, wgrad_event,
                   wgrad_gemm, wgrad_join)

_f = ctypes.c_float

import os as _os

# Code-path switches. They are plain module attributes (tests and the benchmark's baseline arm flip them);
# the only one read from the environment is the memory cap below.
# head_dim 128 / 64 attention with un-fused RoPE runs on the tcgen05 kernels; False keeps everything on the
# mma.sync kernels (A/B comparison).
FLASH_TC = True
FLASH_TC_BWD = True
# dQ from stored dS: the dK/dV kernel writes dS^T (B * QH * Tp^2 bf16, Tp = T rounded up to 128) into a
# workspace that is kept per shape, and dQ becomes a GEMM over it. When the whole batch does not fit the
# limit (``B200_FLASH_DS_WS_GIB``, default 4) the backward runs in chunks of batch elements that do.
FLASH_DQ_GEMM = True
FLASH_DQ_GEMM_MAX_BYTES = int(float(_os.environ.get("B200_FLASH_DS_WS_GIB", "4")) * (1 << 30))
# head_dim 64 on the tcgen05 kernels: the forward and the dK/dV kernel + dQ GEMM are templates on the head dimension.
FLASH_TC_D64 = True


def flash_tc_forward_dim(D: int) -> bool:
    """True when the forward for this head_dim runs on the tcgen05 kernels (which take rotated q, k)."""
    return bool(FLASH_TC and (D == 128 or (D == 64 and FLASH_TC_D64)))


# Inverse rotary embedding of dQ and dK inside the epilogues of the tcgen05 backward kernels (fp32
# accumulator rows) instead of a separate in-place pass over the [dK | dQ] columns; the second switch is the
# same for head_dim 64.
FLASH_ROPE_EPILOGUE = True
FLASH_ROPE_EPILOGUE_D64 = True
_ds_ws_cache: dict = {}


def _ds_batch_chunk(B: int, QH: int, T: int) -> int:
    """Batch elements whose dS^T (QH * Tp^2 bf16 each) fit the workspace limit together; 0 if not even one."""
    tp = (T + 127) // 128 * 128
    return min(B, FLASH_DQ_GEMM_MAX_BYTES // (QH * tp * tp * 2))


def _ds_workspace(device, B: int, QH: int, T: int):
    tp = (T + 127) // 128 * 128
    n = B * QH * tp * tp
    if n * 2 > FLASH_DQ_GEMM_MAX_BYTES:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(), n)
    ws = _ds_ws_cache.get(key)
    if ws is None:
        _ds_ws_cache.clear()           # one shape at a time: a training run has one
        ws = _ds_ws_cache[key] = torch.empty(n, dtype=torch.bfloat16, device=device)
    return ws


_fusion_defaults: dict = {}


def set_unfused_baseline(on: bool) -> None:
    """Switch the epilogue fusions and stream overlaps off (``on``) or back to their defaults: rotary
    embedding in the K|Q|V GEMM epilogue and in the attention-backward epilogues, SwiGLU in the gate|value
    GEMM epilogue, the attention backward's delta in the output projection's dgrad epilogue, loss statistics / logit gradients in the LM-head GEMM epilogues, weight-gradient GEMMs on
    a side stream. With all of them off every one of these steps is a separate kernel on one stream: the
    plain path the benchmark measures the product against."""
    from . import gemm as _g
    global FLASH_ROPE_EPILOGUE, FLASH_ROPE_EPILOGUE_D64, SWIGLU_EPILOGUE, CE_EPILOGUE, DELTA_EPILOGUE
    if not _fusion_defaults:
        _fusion_defaults.update(rope=_g.GEMM_ROPE_EPILOGUE, wgrad=_g.WGRAD_OVERLAP, frope=FLASH_ROPE_EPILOGUE,
                                frope64=FLASH_ROPE_EPILOGUE_D64, swiglu=SWIGLU_EPILOGUE, ce=CE_EPILOGUE,
                                delta=DELTA_EPILOGUE)
    d = _fusion_defaults
    _g.GEMM_ROPE_EPILOGUE = False if on else d["rope"]
    _g.WGRAD_OVERLAP = False if on else d["wgrad"]
    FLASH_ROPE_EPILOGUE = False if on else d["frope"]
    FLASH_ROPE_EPILOGUE_D64 = False if on else d["frope64"]
    SWIGLU_EPILOGUE = False if on else d["swiglu"]
    CE_EPILOGUE = False if on else d["ce"]
    DELTA_EPILOGUE = False if on else d["delta"]


# SwiGLU inside the epilogue of the gate|value projection, and the loss statistics / logit gradients inside
# the epilogues of the LM-head GEMMs (see ``gemm.gemm_swiglu`` / ``gemm.gemm_ce_stats`` / ``gemm.gemm_ce_dlogits``).
SWIGLU_EPILOGUE = True
CE_EPILOGUE = True
# delta = rowsum(dO * O) of the attention backward inside the epilogue of the output projection's dgrad GEMM
# (``gemm.gemm_delta``) instead of a pass of its own.
DELTA_EPILOGUE = True


def _lib():
    native.status_tensor()
    return native.lib()


def _bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError("native kernels take bf16 tensors")


# --------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6):
    """y = x * rsqrt(mean(x^2) + eps) * gamma over the last dim. Returns (y, rstd[M] fp32)."""
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    M = x2.shape[0]
    if not x.is_cuda:
        xf = x2.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        y = (xf * rstd[:, None] * gamma.float()).to(x.dtype)
        return y.view(x.shape), rstd
    _bf16(x, gamma)
    x2 = x2.contiguous()
    y = torch.empty_like(x2)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    native.check(_lib().b200_rmsnorm_fwd(native.ptr(x2), native.ptr(gamma), native.ptr(y), native.ptr(rstd),
                                         M, H, _f(eps), native.stream_ptr()), "rmsnorm_fwd")
    native.bump()
    return y.view(x.shape), rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, rstd: torch.Tensor,
                add: torch.Tensor | None = None):
    """Returns (dx (+ add), dgamma). ``x`` is the layer INPUT; ``add`` is the residual gradient."""
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    dy2 = dy.reshape(-1, H)
    M = x2.shape[0]
    if not x.is_cuda:
        xf, dyf, g = x2.float(), dy2.float(), gamma.float()
        xh = xf * rstd[:, None]
        wdy = dyf * g
        dx = rstd[:, None] * (wdy - xh * (wdy * xh).mean(-1, keepdim=True))
        if add is not None:
            dx = dx + add.reshape(-1, H).float()
        dgamma = (dyf * xh).sum(0)
        return dx.to(x.dtype).view(x.shape), dgamma.to(gamma.dtype)
    _bf16(dy, x, gamma, add)
    x2 = x2.contiguous()
    dy2 = dy2.contiguous()
    add2 = add.reshape(-1, H).contiguous() if add is not None else None
    dx = torch.empty_like(x2)
    dgamma = torch.empty_like(gamma)
    lib = _lib()
    rows = lib.b200_rmsnorm_bwd_partial_rows(M)
    partial = torch.empty((rows, H), dtype=torch.float32, device=x.device)
    native.check(lib.b200_rmsnorm_bwd(native.ptr(dy2), native.ptr(x2), native.ptr(gamma), native.ptr(rstd),
                                      native.ptr(add2), native.ptr(dx), native.ptr(dgamma), native.ptr(partial),
                                      M, H, 0, native.stream_ptr()), "rmsnorm_bwd")
    native.bump(2)
    return dx.view(x.shape), dgamma


# --------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(gate_val: torch.Tensor) -> torch.Tensor:
    """gate_val [M, 2I] = [gate | value] -> silu(gate) * value  [M, I]."""
    M, two_i = gate_val.shape
    I = two_i // 2
    if not gate_val.is_cuda:
        g, v = gate_val[:, :I].float(), gate_val[:, I:].float()
        return (torch.nn.functional.silu(g) * v).to(gate_val.dtype)
    _bf16(gate_val)
    assert gate_val.stride(1) == 1
    act = torch.empty((M, I), dtype=gate_val.dtype, device=gate_val.device)
    native.check(_lib().b200_swiglu_fwd(native.ptr(gate_val), native.ptr(act), M, I, gate_val.stride(0),
                                        native.stream_ptr()), "swiglu_fwd")
    native.bump()
    return act


def swiglu_bwd(dact: torch.Tensor, gate_val: torch.Tensor) -> torch.Tensor:
    M, two_i = gate_val.shape
    I = two_i // 2
    if not gate_val.is_cuda:
        g, v, d = gate_val[:, :I].float(), gate_val[:, I:].float(), dact.float()
        s = torch.sigmoid(g)
        dg = d * v * s * (1 + g * (1 - s))
        dv = d * g * s
        return torch.cat([dg, dv], 1).to(gate_val.dtype)
    _bf16(dact, gate_val)
    assert gate_val.is_contiguous()
    dact = dact.contiguous()
    out = torch.empty_like(gate_val)
    native.check(_lib().b200_swiglu_bwd(native.ptr(dact), native.ptr(gate_val), native.ptr(out), M, I,
                                        gate_val.stride(0), native.stream_ptr()), "swiglu_bwd")
    native.bump()
    return out


# --------------------------------------------------------------------------- RoPE
_rope_cache: dict = {}


def rope_table(T: int, D: int, base: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [T, D/2] fp32 with freq_j = base^(-2j/D)."""
    device = torch.device(device)
    key = (T, D, float(base), device.type, device.index)
    hit = _rope_cache.get(key)
    if hit is not None:
        return hit
    if device.type != "cuda":
        j = torch.arange(D // 2, dtype=torch.float32)
        freq = torch.pow(torch.tensor(float(base)), -2.0 * j / D)
        ang = torch.arange(T, dtype=torch.float32)[:, None] * freq[None, :]
        res = (torch.cos(ang), torch.sin(ang))
    else:
        cs = torch.empty((T, D // 2), dtype=torch.float32, device=device)
        sn = torch.empty_like(cs)
        native.check(_lib().b200_rope_table(native.ptr(cs), native.ptr(sn), T, D, _f(base), native.stream_ptr()),
                     "rope_table")
        native.bump()
        res = (cs, sn)
    _rope_cache[key] = res
    return res


def rope_inplace(buf: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, T: int, nheads: int, D: int,
                 col0: int = 0, pos0: int = 0, inverse: bool = False) -> torch.Tensor:
    """Rotate ``nheads`` heads of width D starting at column ``col0`` of a [M, ld] buffer in place.

    Token m sits at position pos0 + (m % T). Half-split pairing (j, j + D/2).
    """
    M = buf.shape[0]
    if not buf.is_cuda:
        pos = pos0 + (torch.arange(M) % T)
        c = cos[pos][:, None, :]
        s = sin[pos][:, None, :] * (-1.0 if inverse else 1.0)
        v = buf[:, col0:col0 + nheads * D].reshape(M, nheads, D).float()
        x1, x2 = v[..., :D // 2], v[..., D // 2:]
        out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).reshape(M, nheads * D)
        buf[:, col0:col0 + nheads * D] = out.to(buf.dtype)
        return buf
    _bf16(buf)
    assert buf.stride(1) == 1
    native.check(_lib().b200_rope_inplace(native.ptr(buf), native.ptr(cos), native.ptr(sin), M, T, nheads, D,
                                          buf.stride(0), col0, pos0, int(inverse), native.stream_ptr()),
                 "rope_inplace")
    native.bump()
    return buf


# --------------------------------------------------------------------------- embedding
def embedding_fwd(W: torch.Tensor, idx: torch.Tensor, pad_id: int) -> torch.Tensor:
    """out[m] = W[idx[m]], zeros where idx == pad_id. idx is int32 [M]. On CUDA an id >= W.shape[0] reads
    nothing (zeros) and sets native status error 4 (kernel id 401; 402 in the backward)."""
    M = idx.numel()
    H = W.shape[1]
    if not W.is_cuda:
        out = W[idx.long().clamp_min(0)]
        out = out * (idx != pad_id).to(out.dtype)[:, None]
        return out
    _bf16(W)
    assert idx.dtype == torch.int32 and W.is_contiguous()
    out = torch.empty((M, H), dtype=W.dtype, device=W.device)
    native.check(_lib().b200_embedding_fwd(native.ptr(W), native.ptr(idx), native.ptr(out), M, H, pad_id,
                                           W.shape[0], native.stream_ptr()), "embedding_fwd")
    native.bump()
    return out


def embedding_bwd(dW: torch.Tensor, idx: torch.Tensor, dout: torch.Tensor, pad_id: int) -> torch.Tensor:
    """dW[idx[m]] += dout[m] for idx != pad_id (dW is bf16 or fp32, updated in place)."""
    M = idx.numel()
    H = dW.shape[1]
    if not dW.is_cuda:
        keep = idx != pad_id
        dW.index_add_(0, idx[keep].long(), dout[keep].to(dW.dtype))
        return dW
    _bf16(dout)
    assert idx.dtype == torch.int32 and dW.is_contiguous()
    dout = dout.contiguous()
    native.check(_lib().b200_embedding_bwd(native.ptr(dW), native.ptr(idx), native.ptr(dout), M, H, pad_id,
                                           dW.shape[0], int(dW.dtype == torch.float32), native.stream_ptr()),
                 "embedding_bwd")
    native.bump()
    return dW


def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if not a.is_cuda:
        r = a + b
        if out is not None:
            out.copy_(r)
            return out
        return r
    _bf16(a, b)
    a = a.contiguous()
    b = b.contiguous()
    if out is None:
        out = torch.empty_like(a)
    native.check(_lib().b200_add_bf16(native.ptr(a), native.ptr(b), native.ptr(out), ctypes.c_longlong(a.numel()),
                                      native.stream_ptr()), "add_bf16")
    native.bump()
    return out


# --------------------------------------------------------------------------- dropout (bit-packed mask)
def _s64(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(z: torch.Tensor, k: int) -> torch.Tensor:
    return (z >> k) & ((1 << (64 - k)) - 1)


def _drop_keep_reference(n: int, seed: int, offset: int, p: float, device="cpu") -> torch.Tensor:
    """keep[i] of the dropout kernels as a bool tensor: a 64-bit mix of (seed, (offset + i) / 4) gives four
    16-bit lanes, element i keeps when its lane >= round(p * 65536)."""
    i = torch.arange(n, dtype=torch.int64, device=device) + int(offset)
    z = (i >> 2) * _s64(0xD1342543DE82EF95)
    z = z ^ _s64(seed)
    z = z + _s64(0x9E3779B97F4A7C15)
    z = (z ^ _lsr(z, 30)) * _s64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _s64(0x94D049BB133111EB)
    z = z ^ _lsr(z, 31)
    lane = (z >> ((i & 3) * 16)) & 0xFFFF
    return lane >= int(p * 65536.0 + 0.5)


def _packbits(keep: torch.Tensor) -> torch.Tensor:
    """bool [n] -> uint8 [(n + 7) / 8], first element in the most significant bit (numpy.packbits order)."""
    n = keep.numel()
    pad = (-n) % 8
    k = torch.cat([keep.reshape(-1), keep.new_zeros(pad)]).reshape(-1, 8).to(torch.int32)
    w = torch.tensor([128, 64, 32, 16, 8, 4, 2, 1], dtype=torch.int32, device=keep.device)
    return (k * w).sum(1).to(torch.uint8)


def _unpackbits(mask: torch.Tensor, n: int) -> torch.Tensor:
    w = torch.tensor([128, 64, 32, 16, 8, 4, 2, 1], dtype=torch.int32, device=mask.device)
    return ((mask.to(torch.int32)[:, None] & w) != 0).reshape(-1)[:n]


def dropout_fwd(x: torch.Tensor, p: float, seed: int, offset: int):
    """Inverted dropout: returns (x * keep / (1 - p), mask) where ``mask`` holds one BIT per element (uint8
    [(n + 7) / 8]). The keep pattern is a pure function of (seed, offset + element index); ``offset`` must be a
    multiple of 8 and callers advance it by the padded element count of every call."""
    n = x.numel()
    if not x.is_cuda:
        keep = _drop_keep_reference(n, seed, offset, p, x.device).view(x.shape)
        return (x * keep.to(x.dtype) * (1.0 / (1.0 - p))).to(x.dtype), _packbits(keep)
    assert x.dtype in (torch.bfloat16, torch.float32)
    x = x.contiguous()
    out = torch.empty_like(x)
    mask = torch.empty((n + 7) // 8, dtype=torch.uint8, device=x.device)
    native.check(_lib().b200_dropout_fwd(native.ptr(x), native.ptr(out), native.ptr(mask), ctypes.c_longlong(n),
                                         int(x.dtype == torch.float32), ctypes.c_ulonglong(seed & ((1 << 64) - 1)),
                                         ctypes.c_ulonglong(offset), _f(p), native.stream_ptr()), "dropout_fwd")
    native.bump()
    return out, mask


def dropout_bwd(dout: torch.Tensor, mask: torch.Tensor, p: float) -> torch.Tensor:
    """dout * keep / (1 - p) with ``keep`` read from the packed mask of ``dropout_fwd``."""
    n = dout.numel()
    if not dout.is_cuda:
        keep = _unpackbits(mask, n).view(dout.shape)
        return (dout * keep.to(dout.dtype) * (1.0 / (1.0 - p))).to(dout.dtype)
    assert dout.dtype in (torch.bfloat16, torch.float32) and mask.dtype == torch.uint8
    dout = dout.contiguous()
    out = torch.empty_like(dout)
    native.check(_lib().b200_dropout_bwd(native.ptr(dout), native.ptr(mask), native.ptr(out), ctypes.c_longlong(n),
                                         int(dout.dtype == torch.float32), _f(p), native.stream_ptr()), "dropout_bwd")
    native.bump()
    return out


# --------------------------------------------------------------------------- flash attention
def _strides3(t: torch.Tensor) -> list[int]:
    """(batch, token, head) element strides of a [B, T, heads, D] view."""
    assert t.dim() == 4 and t.stride(3) == 1
    return [t.stride(0), t.stride(1), t.stride(2)]


def _attn_reference(q, k, v, valid_len, scale, cos, sin):
    """fp32 dense restatement on [B, T, heads, D] views; returns (o, lse, probs, q_rot, k_rot)."""
    B, T, QH, D = q.shape
    KVH = k.shape[2]
    R = QH // KVH
    qf, kf, vf = q.float(), k.float(), v.float()
    if cos is not None:
        def rot(x):
            c, s = cos[:T][None, :, None, :], sin[:T][None, :, None, :]
            x1, x2 = x[..., :D // 2], x[..., D // 2:]
            return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
        qf, kf = rot(qf), rot(kf)
    kx = kf.repeat_interleave(R, dim=2)
    vx = vf.repeat_interleave(R, dim=2)
    s = torch.einsum("bthd,bshd->bhts", qf, kx) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()[None, None]
    if valid_len is not None:
        keyok = torch.arange(T, device=q.device)[None, :] < valid_len[:, None]
        mask = mask & keyok[:, None, None, :]
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum("bhts,bshd->bthd", p, vx)
    return o, lse, p, qf, kf


def _attn_bwd_reference(dout, q, k, v, o, valid_len, scale, cos, sin, unrotate=None, out=None, p_drop=None):
    """Dense fp32 restatement of the attention backward on [B, T, heads, D] views, on whatever device the
    tensors live (the CPU body of ``flash_attn_bwd`` and the dense verification path of the attention layer).
    ``cos`` / ``sin``: q and k are un-rotated and rotated here; ``unrotate``: they are rotated already and the
    gradients are rotated back. ``p_drop``: a dropout layer whose last forward masked the attention
    probabilities (its packed mask is consumed here)."""
    B, T, QH, D = q.shape
    KVH = k.shape[2]
    R = QH // KVH
    _, _, p, qf, kf = _attn_reference(q, k, v, valid_len, scale, cos, sin)
    dof = dout.float()
    vx = v.float().repeat_interleave(R, dim=2)
    kx = kf.repeat_interleave(R, dim=2)
    if p_drop is not None and p_drop.mask is not None:
        # o = (p * keep / (1 - p_drop)) v: dV sees the dropped probabilities, dP comes back through the mask,
        # and the softmax Jacobian needs sum_s p dP itself (o was not formed from p)
        dvx = torch.einsum("bhts,bthd->bshd", p_drop.reapply(p), dof)
        dp = p_drop.backward(torch.einsum("bthd,bshd->bhts", dof, vx))
        delta = (p * dp).sum(-1)                                    # [B, QH, T]
    else:
        dvx = torch.einsum("bhts,bthd->bshd", p, dof)
        dp = torch.einsum("bthd,bshd->bhts", dof, vx)
        delta = (dof * o.float()).sum(-1).permute(0, 2, 1)          # [B, QH, T]
    ds = p * (dp - delta[..., None]) * scale
    dqf = torch.einsum("bhts,bshd->bthd", ds, kx)
    dkx = torch.einsum("bhts,bthd->bshd", ds, qf)
    dk_ = dkx.reshape(B, T, KVH, R, D).sum(3)
    dv_ = dvx.reshape(B, T, KVH, R, D).sum(3)
    for tabs in ((cos, sin), unrotate):
        if tabs is not None and tabs[0] is not None:
            c = tabs[0][:T][None, :, None, :].float()
            sn = tabs[1][:T][None, :, None, :].float()

            def unrot(x):
                y1, y2 = x[..., :D // 2], x[..., D // 2:]
                return torch.cat([y1 * c + y2 * sn, y2 * c - y1 * sn], -1)
            dqf, dk_ = unrot(dqf), unrot(dk_)
    res = (dqf.to(q.dtype), dk_.to(q.dtype), dv_.to(q.dtype))
    if out is not None:
        for dst, src in zip(out, res):
            dst.copy_(src)
        return out
    return res


def flash_attn_fwd(q, k, v, *, valid_len=None, scale=None, rope=None):
    """Causal GQA attention. q [B,T,QH,D], k/v [B,T,KVH,D] (any strides with unit last stride).

    ``rope`` = (cos, sin) tables [>=T, D/2] rotates Q and K inside the kernel. Returns
    (o [B,T,QH,D] contiguous, lse [B,QH,T] fp32).
    """
    B, T, QH, D = q.shape
    KVH = k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    cos, sin = rope if rope is not None else (None, None)
    if not q.is_cuda:
        o, lse, _, _, _ = _attn_reference(q, k, v, valid_len, scale, cos, sin)
        return o.to(q.dtype).contiguous(), lse
    _bf16(q, k, v)
    o = torch.empty((B, T, QH, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, QH, T), dtype=torch.float32, device=q.device)
    strides = _strides3(q) + _strides3(k) + _strides3(v) + _strides3(o)
    if cos is None and flash_tc_forward_dim(D):
        # tcgen05 / TMEM kernel (inputs already rotated)
        arr = (ctypes.c_longlong * 12)(*strides)
        native.check(_lib().b200_flash_fwd_tc3(native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o),
                                               native.ptr(lse), native.ptr(valid_len), arr, B, T, QH, KVH, D,
                                               _f(scale), native.stream_ptr()), "flash_fwd_tc3")
        native.bump()
        return o, lse
    arr = (ctypes.c_longlong * 24)(*(strides + [0] * 12))
    native.check(_lib().b200_flash_fwd(native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(lse),
                                       native.ptr(valid_len), native.ptr(cos), native.ptr(sin), arr,
                                       B, T, QH, KVH, D, _f(scale), native.stream_ptr()), "flash_fwd")
    native.bump()
    return o, lse


def set_flash_bwd_wide(on: bool) -> bool:
    """head_dim 128: run the dK/dV kernel with 128-query iterations and interleaved products (default), or
    (``on`` False) the kernel with double-buffered 64-query iterations that head_dim 64 uses. Returns the
    previous setting. For A/B runs and tests."""
    return bool(_lib().b200_flash_bwd_wide(1 if on else 0))


def flash_bwd_wide_active() -> bool:
    """True when head_dim 128 runs the dK/dV kernel with 128-query iterations on the current device: switched on
    and its shared memory (all but 872 bytes of an SM's) fits behind the kernel's dynamic shared-memory base."""
    return bool(_lib().b200_flash_bwd_wide_active())


def set_flash_bwd_pairing(mode: int) -> int:
    """Key-tile pairing of the dK/dV kernels: -1 (default) pairs tiles i and n - 1 - i in one CTA when there are
    between one and three key tiles per SM, 0 never, 1 always. Returns the previous value. For A/B runs and tests."""
    return int(_lib().b200_flash_bwd_pairing(int(mode)))


def flash_delta(o: torch.Tensor, dout: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """``delta[b, h, t] = sum_d dout * o`` for [B, T, heads, D] bf16 tensors (fp32 result, [B, heads, T]): the
    stand-alone form of what ``gemm.gemm_delta`` leaves from the output projection's dgrad epilogue."""
    B, T, QH, D = o.shape
    arr6 = (ctypes.c_longlong * 6)(*(_strides3(o) + _strides3(dout)))
    native.check(_lib().b200_flash_delta(native.ptr(o), native.ptr(dout), native.ptr(delta), arr6, B, T, QH, D,
                                         native.stream_ptr()), "flash_delta")
    native.bump()
    return delta


def flash_bwd_can_unrotate(q: torch.Tensor) -> bool:
    """True when ``flash_attn_bwd(..., unrotate=...)`` applies the inverse rotary embedding inside the
    attention-backward kernels (tcgen05 path: head_dim 128, or head_dim 64 with its dS workspace) for this
    tensor [B, T, heads, D]."""
    if not (q.is_cuda and FLASH_TC and FLASH_TC_BWD and FLASH_ROPE_EPILOGUE):
        return False
    D = q.shape[-1]
    if D == 128:
        return True
    return bool(D == 64 and FLASH_ROPE_EPILOGUE_D64 and FLASH_TC_D64 and FLASH_DQ_GEMM
                and _ds_batch_chunk(q.shape[0], q.shape[2], q.shape[1]) >= 1)


def flash_attn_bwd(dout, q, k, v, o, lse, *, valid_len=None, scale=None, rope=None, out=None, unrotate=None,
                   delta=None):
    """Gradients (dq, dk, dv) w.r.t. the UN-rotated q, k and v.

    ``rope=(cos, sin)``: q and k are given un-rotated and rotated on the fly. ``unrotate=(cos, sin)``: q and
    k are given ROTATED (``rope`` must be None) and dq, dk are un-rotated in the kernels' epilogues - only
    where ``flash_bwd_can_unrotate`` holds (and in the CPU restatement). ``out`` may give three
    preallocated [B,T,heads,D] views (e.g. slices of a packed d(KQV) buffer) to write into. ``delta``
    ([B, q heads, T] fp32, ``sum_d dout * o``): already computed by the caller (``gemm.gemm_delta``); used by the
    tcgen05 path, which otherwise computes it with a kernel of its own.
    """
    if unrotate is not None and rope is not None:
        raise ValueError("flash_attn_bwd: rope and unrotate are exclusive")
    B, T, QH, D = q.shape
    KVH = k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    cos, sin = rope if rope is not None else (None, None)
    if not q.is_cuda:
        return _attn_bwd_reference(dout, q, k, v, o, valid_len, scale, cos, sin, unrotate, out)
    _bf16(dout, q, k, v, o)
    if dout.stride(3) != 1:
        dout = dout.contiguous()
    if out is None:
        dq = torch.empty((B, T, QH, D), dtype=q.dtype, device=q.device)
        dk_ = torch.empty((B, T, KVH, D), dtype=q.dtype, device=q.device)
        dv_ = torch.empty((B, T, KVH, D), dtype=q.dtype, device=q.device)
    else:
        dq, dk_, dv_ = out
    have_delta = delta is not None
    if have_delta:
        assert delta.shape == (B, QH, T) and delta.dtype == torch.float32 and delta.is_contiguous()
    else:
        delta = torch.empty((B, QH, T), dtype=torch.float32, device=q.device)
    if unrotate is not None and not flash_bwd_can_unrotate(q):
        raise ValueError("flash_attn_bwd: unrotate= is only fused on the tcgen05 path (see flash_bwd_can_unrotate)")
    # Batch elements per call whose dS^T workspace stays within the limit; when not even one fits, KV-head
    # groups of one batch element per call (kc, 0: not even one group). head_dim 64 has the tcgen05
    # backward only in the form with that workspace (dK/dV kernel + dQ GEMM).
    bc = _ds_batch_chunk(B, QH, T) if (FLASH_DQ_GEMM and (D == 128 or FLASH_TC_D64)) else 0
    kc = 0
    if bc == 0 and FLASH_DQ_GEMM and (D == 128 or FLASH_TC_D64):
        kc = min(KVH, _ds_batch_chunk(KVH, QH // KVH, T))       # a KV-head group holds QH / KVH query heads
    if cos is None and FLASH_TC and FLASH_TC_BWD and (D == 128 or (D == 64 and (bc >= 1 or kc >= 1))):
        # tcgen05 / TMEM kernels (q, k already rotated; dq, dk are w.r.t. the rotated tensors)
        if not have_delta:
            flash_delta(o, dout, delta)
        s21 = (_strides3(q) + _strides3(k) + _strides3(v) + _strides3(dout) + _strides3(dq) + _strides3(dk_) +
               _strides3(dv_))
        arr21 = (ctypes.c_longlong * 21)(*s21)
        R = QH // KVH
        if bc >= 1:
            ws = _ds_workspace(q.device, bc, QH, T)
            chunks = [(b0, min(b0 + bc, B), 0, KVH) for b0 in range(0, B, bc)]
        elif kc >= 1:
            ws = _ds_workspace(q.device, 1, kc * R, T)
            chunks = [(b0, b0 + 1, g0, min(g0 + kc, KVH)) for b0 in range(B) for g0 in range(0, KVH, kc)]
        else:
            ws, chunks = None, [(0, B, 0, KVH)]
        ucos, usin = unrotate if unrotate is not None else (None, None)
        if ucos is not None:
            assert ucos.dtype == torch.float32 and usin.dtype == torch.float32 and ucos.is_contiguous() \
                and usin.is_contiguous() and ucos.shape[0] >= T and ucos.shape[1] == D // 2
            from .gemm import rope_tables_transposed
            ucos, usin = rope_tables_transposed(ucos, usin)[:2]
        uld = ucos.shape[1] if ucos is not None else 0
        for b0, b1, g0, g1 in chunks:       # slices along batch and heads keep every stride
            whole = b1 - b0 == B and g1 - g0 == KVH

            def part(t, kind):      # kind: 0 = [B] vector, 1 = [B, T, kv heads, D], 2 = [B, T, q heads, D], 3 = [B, q heads, T]
                if whole or t is None:
                    return t
                if kind == 0:
                    return t[b0:b1]
                if kind == 1:
                    return t[b0:b1, :, g0:g1]
                if kind == 2:
                    return t[b0:b1, :, g0 * R:g1 * R]
                return t[b0:b1, g0 * R:g1 * R]       # contiguous: head slices only come with one batch element
            native.check(_lib().b200_flash_bwd_tc(native.ptr(part(q, 2)), native.ptr(part(k, 1)), native.ptr(part(v, 1)),
                                                  native.ptr(part(dout, 2)), native.ptr(part(lse, 3)),
                                                  native.ptr(part(delta, 3)), native.ptr(part(dq, 2)),
                                                  native.ptr(part(dk_, 1)), native.ptr(part(dv_, 1)),
                                                  native.ptr(part(valid_len, 0)),
                                                  arr21, b1 - b0, T, (g1 - g0) * R, g1 - g0, D, _f(scale), native.ptr(ws),
                                                  native.ptr(ucos), native.ptr(usin), uld, native.stream_ptr()),
                         "flash_bwd_tc")
        native.bump(2 * len(chunks))
        return dq, dk_, dv_
    strides = (_strides3(q) + _strides3(k) + _strides3(v) + _strides3(o) + _strides3(dout) +
               _strides3(dq) + _strides3(dk_) + _strides3(dv_))
    arr = (ctypes.c_longlong * 24)(*strides)
    native.check(_lib().b200_flash_bwd(native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(dout),
                                       native.ptr(lse), native.ptr(delta), native.ptr(dq), native.ptr(dk_),
                                       native.ptr(dv_), native.ptr(valid_len), native.ptr(cos), native.ptr(sin), arr,
                                       B, T, QH, KVH, D, _f(scale), native.stream_ptr()), "flash_bwd")
    native.bump(3)
    return dq, dk_, dv_


def decode_attn(q, kcache, vcache, lens, scale=None):
    """One-token attention against a KV cache. q [B,QH,D]; caches [B,KVH,Tmax,D]; lens int32 [B]."""
    B, QH, D = q.shape
    KVH, Tmax = kcache.shape[1], kcache.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if not q.is_cuda:
        R = QH // KVH
        kx = kcache.float().repeat_interleave(R, dim=1)
        vx = vcache.float().repeat_interleave(R, dim=1)
        s = torch.einsum("bhd,bhtd->bht", q.float(), kx) * scale
        ok = torch.arange(Tmax)[None, None, :] < lens[:, None, None]
        s = s.masked_fill(~ok, float("-inf"))
        p = torch.softmax(s, -1)
        return torch.einsum("bht,bhtd->bhd", p, vx).to(q.dtype)
    _bf16(q, kcache, vcache)
    assert q.is_contiguous() and kcache.is_contiguous() and vcache.is_contiguous() and lens.dtype == torch.int32
    out = torch.empty_like(q)
    native.check(_lib().b200_decode_attn(native.ptr(q), native.ptr(kcache), native.ptr(vcache), native.ptr(out),
                                         native.ptr(lens), B, QH, KVH, Tmax, D, _f(scale), native.stream_ptr()),
                 "decode_attn")
    native.bump()
    return out


# --------------------------------------------------------------------------- cross-entropy rows
def ce_stats(logits, targets, rmax, rsum, tlogit, col0: int, first: bool):
    """Fold one fp32 logits chunk [M, C] (vocab ids col0..col0+C) into the running row statistics."""
    M, C = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        mx = lf.max(-1).values
        old = torch.full_like(mx, float("-inf")) if first else rmax.clone()
        new = torch.maximum(old, mx)
        s = torch.exp(lf - new[:, None]).sum(-1)
        olds = torch.zeros_like(s) if first else rsum
        rsum.copy_(olds * torch.exp(old - new) + s)
        rmax.copy_(new)
        t = targets.long() - col0
        hit = (t >= 0) & (t < C)
        rows = torch.nonzero(hit).flatten()
        tlogit[rows] = lf[rows, t[rows]]
        return
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and targets.dtype == torch.int32
    native.check(_lib().b200_ce_stats(native.ptr(logits), native.ptr(targets), native.ptr(rmax), native.ptr(rsum),
                                      native.ptr(tlogit), M, C, logits.stride(0), col0, int(first),
                                      native.stream_ptr()), "ce_stats")
    native.bump()


def ce_loss(rmax, rsum, tlogit, targets, pad_id: int) -> torch.Tensor:
    """Returns a 2-float tensor [sum of row losses over valid rows, number of valid rows]."""
    M = targets.numel()
    if not rmax.is_cuda:
        valid = (targets != pad_id) & (targets >= 0)
        loss = (rmax + torch.log(rsum) - tlogit)[valid].sum()
        return torch.stack([loss, valid.sum().float()])
    out = torch.zeros(2, dtype=torch.float32, device=rmax.device)
    native.check(_lib().b200_ce_loss(native.ptr(rmax), native.ptr(rsum), native.ptr(tlogit), native.ptr(targets),
                                     native.ptr(out), M, pad_id, native.stream_ptr()), "ce_loss")
    native.bump()
    return out


def ce_dlogits(logits, targets, rmax, rsum, loss_cnt, col0: int, pad_id: int, gscale: float, out_dtype):
    """(softmax - onehot) * valid * gscale / n_valid for one logits chunk, in ``out_dtype``."""
    M, C = logits.shape
    if not logits.is_cuda:
        p = torch.exp(logits.float() - rmax[:, None]) / rsum[:, None]
        t = targets.long() - col0
        hit = (t >= 0) & (t < C)
        rows = torch.nonzero(hit).flatten()
        p[rows, t[rows]] -= 1.0
        valid = ((targets != pad_id) & (targets >= 0)).float()
        p = p * (valid * gscale / loss_cnt[1].clamp_min(1.0))[:, None]
        return p.to(out_dtype)
    assert out_dtype == torch.bfloat16
    out = torch.empty((M, C), dtype=torch.bfloat16, device=logits.device)
    native.check(_lib().b200_ce_dlogits(native.ptr(logits), native.ptr(targets), native.ptr(rmax), native.ptr(rsum),
                                        native.ptr(loss_cnt), native.ptr(out), M, C, logits.stride(0), C, col0,
                                        pad_id, _f(gscale), native.stream_ptr()), "ce_dlogits")
    native.bump()
    return out


def ce_merge(pmax: torch.Tensor, psum: torch.Tensor):
    """Merge per-tile row statistics [nt, M] (see ``gemm_ce_stats``) into (rmax [M], rsum [M])."""
    nt, M = pmax.shape
    if not pmax.is_cuda:
        mx = pmax.max(0).values
        return mx, (psum * torch.exp(pmax - mx[None, :])).sum(0)
    rmax = torch.empty(M, dtype=torch.float32, device=pmax.device)
    rsum = torch.empty_like(rmax)
    native.check(_lib().b200_ce_merge(native.ptr(pmax), native.ptr(psum), native.ptr(rmax), native.ptr(rsum), M, nt,
                                      native.stream_ptr()), "ce_merge")
    native.bump()
    return rmax, rsum


def ce_row_coef(rmax, rsum, targets, loss_cnt, pad_id: int, gscale: float):
    """(lse [M], coef [M]) for the logit-gradient epilogue: lse = rmax + log(rsum), coef = valid * gscale / n_valid."""
    M = rmax.numel()
    if not rmax.is_cuda:
        valid = ((targets != pad_id) & (targets >= 0)).float()
        return rmax + torch.log(rsum), valid * gscale / loss_cnt[1].clamp_min(1.0)
    lse = torch.empty(M, dtype=torch.float32, device=rmax.device)
    coef = torch.empty_like(lse)
    native.check(_lib().b200_ce_row_coef(native.ptr(rmax), native.ptr(rsum), native.ptr(targets), native.ptr(loss_cnt),
                                         native.ptr(lse), native.ptr(coef), M, pad_id, _f(gscale), native.stream_ptr()),
                 "ce_row_coef")
    native.bump()
    return lse, coef


# --------------------------------------------------------------------------- optimizer side
def adamw_step(grad, m, v, master, param, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
               max_grad_norm=0.0, stats=None, hyper=None):
    """In-place AdamW on a flat shard: fp32 master/m/v, bf16 (or same-dtype) param written back.

    ``stats`` = device tensor [sum g^2 (unscaled), non-finite flag]: when given, the clip
    coefficient min(1, max_norm / (sqrt(stats[0]) * grad_scale + 1e-6)) is applied and the whole
    update is skipped if stats[1] != 0, both decided on the device. ``hyper`` = device tensor
    [lr, m_corr, v_corr, grad_scale] that overrides the host values of the same names (for launches
    replayed from a CUDA graph).
    """
    m_corr = 1.0 / (1.0 - beta1 ** step)
    v_corr = 1.0 / (1.0 - beta2 ** step)
    n = grad.numel()
    if not grad.is_cuda:
        gmul = grad_scale
        if stats is not None:
            if float(stats[1]) != 0.0:
                return
            if max_grad_norm > 0:
                norm = math.sqrt(float(stats[0])) * grad_scale
                gmul *= min(1.0, max_grad_norm / (norm + 1e-6))
        g = grad.float() * gmul
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        if weight_decay > 0:
            master.mul_(1 - lr * weight_decay)
        master.sub_(lr * (m * m_corr) / (torch.sqrt(v * v_corr) + eps))
        param.copy_(master.to(param.dtype))
        return
    assert param.dtype == torch.bfloat16 and grad.dtype in (torch.bfloat16, torch.float32)
    assert all(t.is_contiguous() for t in (grad, m, v, master, param))
    if hyper is not None:
        native.check(_lib().b200_adamw_dev(native.ptr(grad), int(grad.dtype == torch.float32), native.ptr(m),
                                           native.ptr(v), native.ptr(master), native.ptr(param), ctypes.c_longlong(n),
                                           _f(beta1), _f(beta2), _f(eps), _f(weight_decay), _f(max_grad_norm),
                                           native.ptr(stats), native.ptr(hyper), native.stream_ptr()), "adamw_dev")
        native.bump()
        return
    native.check(_lib().b200_adamw(native.ptr(grad), int(grad.dtype == torch.float32), native.ptr(m), native.ptr(v),
                                   native.ptr(master), native.ptr(param), ctypes.c_longlong(n), _f(lr), _f(beta1),
                                   _f(beta2), _f(eps), _f(weight_decay), _f(m_corr), _f(v_corr), _f(grad_scale),
                                   _f(max_grad_norm), native.ptr(stats), native.stream_ptr()), "adamw")
    native.bump()


def grad_stats(g: torch.Tensor, stats: torch.Tensor) -> None:
    """stats[0] += sum of squares of the finite entries of g; stats[1] = 1 if any is NaN/Inf."""
    if not g.is_cuda:
        gf = g.float()
        fin = torch.isfinite(gf)
        stats[0] += (gf[fin] ** 2).sum()
        if not bool(fin.all()):
            stats[1] = 1.0
        return
    assert g.is_contiguous() and stats.dtype == torch.float32
    native.check(_lib().b200_grad_stats(native.ptr(g), int(g.dtype == torch.float32), ctypes.c_longlong(g.numel()),
                                        native.ptr(stats), native.stream_ptr()), "grad_stats")
    native.bump()


def accumulate(acc: torch.Tensor, g: torch.Tensor, scale: float = 1.0) -> None:
    """acc (fp32) += g * scale."""
    if not acc.is_cuda:
        acc.add_(g.float(), alpha=scale)
        return
    assert acc.dtype == torch.float32 and acc.is_contiguous() and g.is_contiguous()
    native.check(_lib().b200_accumulate(native.ptr(acc), native.ptr(g), int(g.dtype == torch.float32),
                                        ctypes.c_longlong(acc.numel()), _f(scale), native.stream_ptr()), "accumulate")
    native.bump()
