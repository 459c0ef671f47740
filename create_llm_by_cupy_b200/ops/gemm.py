"""bf16 GEMM front end: tcgen05 kernel on CUDA tensors, fp32 torch restatement on CPU tensors.

Replaces the ``cp.matmul`` (cuBLAS) call sites of the reference
(model/fast_layers.py:217,341,420,423,457,458,736,748,794,797,813,815,1328,1351,1435,1464,1471).
"""
from __future__ import annotations

import ctypes

import torch

from . import native

GEMM_OUT_F32 = 1
GEMM_ADD_C = 2
GEMM_WHOLE_TILES = 8      # CTA-pair kernel: do not split the tiles of a part-filled last round

# Code-path switches (module attributes; tests and the benchmark's baseline arm set them).
# "1cta": single-CTA 128x256 tiles; "2cta": CTA pairs (cta_group::2) on 256x256 tiles where the
# problem is large enough, single-CTA otherwise.
GEMM_IMPL = "2cta"
# Tile hand-out of the CTA-pair kernel: 1 = tiles beyond each pair's first come from a device
# counter (pairs that start late draw fewer), 0 = fixed round-robin assignment.
GEMM_DYNAMIC_TILES = 1
_dynamic_applied = None
# 1: when the last round of 256x256 tiles would fill less than half of the CTA pairs, those tiles
# are split into 256x128 halves so that twice as many pairs work on it; 0: whole tiles only.
GEMM_HALF_TILES = 1
_half_applied = None


def set_dynamic_tiles(on: bool) -> None:
    global GEMM_DYNAMIC_TILES
    GEMM_DYNAMIC_TILES = int(on)


def set_half_tiles(on: bool) -> None:
    global GEMM_HALF_TILES
    GEMM_HALF_TILES = int(on)


def _apply_dynamic():
    global _dynamic_applied, _half_applied
    if _dynamic_applied != GEMM_DYNAMIC_TILES:
        native.lib().b200_gemm_2cta_dynamic_tiles(int(GEMM_DYNAMIC_TILES))
        _dynamic_applied = GEMM_DYNAMIC_TILES
    if _half_applied != GEMM_HALF_TILES:
        native.lib().b200_gemm_2cta_half_tiles(int(GEMM_HALF_TILES))
        _half_applied = GEMM_HALF_TILES


def _rowmajor_2d(t: torch.Tensor) -> tuple[torch.Tensor, int]:
    """Return (tensor, pitch) for a 2-D view whose last dim is contiguous; copy if it is not."""
    assert t.dim() == 2
    if t.stride(1) != 1 or (t.size(0) > 1 and t.stride(0) < t.size(1)):
        t = t.contiguous()
    return t, (t.stride(0) if t.size(0) > 1 else max(t.size(1), t.stride(0)))


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         out: torch.Tensor | None = None, add: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, alpha: float = 1.0, bn: int = 0,
         max_ctas: int = 0, force_fallback: bool = False, impl: str | None = None) -> torch.Tensor:
    """``out = alpha * op(a) @ op(b) (+ add)``.

    ``a`` is ``[M, K]`` (``[K, M]`` with ``trans_a``); ``b`` is ``[K, N]`` (``[N, K]`` with
    ``trans_b``). Inputs are bf16 on CUDA; ``out``/``add`` are bf16 or fp32 (same dtype) and
    ``add`` may alias ``out`` (accumulation). Accumulation is fp32 in TMEM.
    """
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    Kb, N = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: inner dims differ ({K} vs {Kb})")
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else (add.dtype if add is not None else a.dtype)

    if not a.is_cuda:
        af = a.float().t() if trans_a else a.float()
        bf = b.float().t() if trans_b else b.float()
        res = (af @ bf) * alpha
        if add is not None:
            res = res + add.float()
        res = res.to(out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm: CUDA operands must be bf16")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("gemm: out dtype must be bf16 or fp32")
    a, lda = _rowmajor_2d(a)
    b, ldb = _rowmajor_2d(b)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.dim() == 2 and out.shape == (M, N) and out.stride(1) == 1 and out.dtype == out_dtype
    ldd = out.stride(0) if M > 1 else max(N, out.stride(0))
    flags = GEMM_OUT_F32 if out_dtype == torch.float32 else 0
    ldc = 0
    if add is not None:
        assert add.shape == (M, N) and add.stride(1) == 1 and add.dtype == out_dtype
        ldc = add.stride(0) if M > 1 else max(N, add.stride(0))
        flags |= GEMM_ADD_C
    native.status_tensor()
    impl = impl or GEMM_IMPL
    if (impl == "2cta" and not force_fallback and bn == 0 and max_ctas == 0 and M >= 256 and N >= 256
            and lda % 8 == 0 and ldb % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0):
        _apply_dynamic()
        # Half tiles shorten the tail of a GEMM that has the GPU to itself. While weight-gradient GEMMs
        # are in flight on the side stream the tail is filled by the other kernel's CTAs, and narrower
        # tiles only cost efficiency (measured on the 1.3 B step: 1.1 ms faster alone, 1.2 ms slower beside).
        if _wgrad_pending.get(a.device.index, False):
            flags |= GEMM_WHOLE_TILES
        rc = native.lib().b200_gemm_bf16_2cta(
            native.ptr(a), native.ptr(b), native.ptr(out), native.ptr(add),
            M, N, K, lda, ldb, ldd, ldc, int(trans_a), int(not trans_b), flags,
            ctypes.c_float(alpha), native.stream_ptr())
        native.check(rc, "b200_gemm_bf16_2cta")
        native.bump()
        return out
    rc = native.lib().b200_gemm_bf16(
        native.ptr(a), native.ptr(b), native.ptr(out), native.ptr(add),
        M, N, K, lda, ldb, ldd, ldc, int(trans_a), int(not trans_b), flags,
        ctypes.c_float(alpha), bn, max_ctas, int(force_fallback), native.stream_ptr())
    native.check(rc, "b200_gemm_bf16")
    native.bump()
    return out


# Rotary embedding in the epilogue of the CTA-pair kernel instead of an in-place pass over the output.
GEMM_ROPE_EPILOGUE = True


_rope_t_cache: dict = {}


def rope_tables_transposed(cos: torch.Tensor, sin: torch.Tensor):
    """([D/2, T] cos, [D/2, T] sin) copies of the [T, D/2] rotary tables, cached per table. The kernels'
    epilogues own one row (position) per thread, so a warp reads consecutive words from this layout."""
    key = (cos.data_ptr(), sin.data_ptr(), tuple(cos.shape))
    tt = _rope_t_cache.get(key)
    if tt is None:
        if len(_rope_t_cache) > 16:
            _rope_t_cache.clear()
        tt = _rope_t_cache[key] = (cos.t().contiguous(), sin.t().contiguous(), cos, sin)   # keeps the sources alive
    return tt


def gemm_rope_fusable(a: torch.Tensor, b: torch.Tensor, head_dim: int, rope_cols: int) -> bool:
    """True when ``gemm_rope(a, b, ...)`` (``a`` [M, K], ``b`` [K, N], both row-major bf16) runs with the
    rotation fused into the GEMM epilogue."""
    if not (GEMM_ROPE_EPILOGUE and a.is_cuda and GEMM_IMPL == "2cta" and head_dim in (64, 128)):
        return False
    M, N = a.shape[0], b.shape[1]
    return bool(a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and M >= 256 and N >= 256 and N % 8 == 0
                and rope_cols % head_dim == 0 and 0 < rope_cols <= N
                and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0
                and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)


def gemm_rope(a: torch.Tensor, b: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, T: int, head_dim: int,
              rope_cols: int) -> torch.Tensor:
    """``a @ b`` whose first ``rope_cols`` output columns are heads of width ``head_dim`` rotated by the
    rotary embedding of position ``row % T`` (half-split pairing, tables fp32 [>= T, head_dim / 2]).
    Only where ``gemm_rope_fusable`` holds."""
    M, K = a.shape
    N = b.shape[1]
    assert gemm_rope_fusable(a, b, head_dim, rope_cols)
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    assert cos.shape[0] >= T and cos.shape[1] == head_dim // 2
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    native.status_tensor()
    _apply_dynamic()
    flags = GEMM_WHOLE_TILES if _wgrad_pending.get(a.device.index, False) else 0
    # the epilogue reads the tables transposed ([head_dim / 2][positions]): a thread owns a row, so a warp
    # then reads consecutive words
    tt = rope_tables_transposed(cos, sin)
    rc = native.lib().b200_gemm_bf16_2cta_rope(
        native.ptr(a), native.ptr(b), native.ptr(out), M, N, K, a.stride(0), b.stride(0), N, 0, 1, flags,
        native.ptr(tt[0]), native.ptr(tt[1]), T, tt[0].shape[1], rope_cols, head_dim, native.stream_ptr())
    native.check(rc, "b200_gemm_bf16_2cta_rope")
    native.bump()
    return out


def _tma_ok(*ts) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
               and t.data_ptr() % 16 == 0 for t in ts)


def _whole_tiles_flag(device) -> int:
    return GEMM_WHOLE_TILES if _wgrad_pending.get(device.index, False) else 0


def gemm_swiglu_fusable(x: torch.Tensor, w_gate_val: torch.Tensor) -> bool:
    """True when ``gemm_swiglu(x, w_gate_val)`` runs as one kernel (``x`` [M, K], ``w_gate_val`` [K, 2 I], bf16)."""
    if not (x.is_cuda and GEMM_IMPL == "2cta" and _tma_ok(x, w_gate_val)):
        return False
    I = w_gate_val.shape[1] // 2
    return x.shape[0] >= 256 and I >= 128 and w_gate_val.shape[1] == 2 * I and I % 8 == 0


def gemm_swiglu(x: torch.Tensor, w_gate_val: torch.Tensor, keep_gv: bool = True):
    """``gv = x @ [W_gate | W_value]`` and ``act = silu(gate) * value`` from ONE GEMM whose epilogue applies the
    activation to the fp32 accumulator (a tile holds 128 gate columns beside the matching 128 value columns).
    Returns ``(gv [M, 2 I] or None, act [M, I])``; ``gv`` is only written when ``keep_gv`` (the backward reads it).
    Only where ``gemm_swiglu_fusable`` holds."""
    M, K = x.shape
    I = w_gate_val.shape[1] // 2
    assert gemm_swiglu_fusable(x, w_gate_val)
    act = torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
    gv = torch.empty((M, 2 * I), dtype=torch.bfloat16, device=x.device) if keep_gv else None
    native.status_tensor()
    _apply_dynamic()
    rc = native.lib().b200_gemm_bf16_2cta_swiglu(
        native.ptr(x), native.ptr(w_gate_val), native.ptr(gv), native.ptr(act), M, I, K, x.stride(0),
        w_gate_val.stride(0), 2 * I, I, _whole_tiles_flag(x.device), native.stream_ptr())
    native.check(rc, "b200_gemm_bf16_2cta_swiglu")
    native.bump()
    return gv, act


def gemm_swiglu_bwd_fusable(dout: torch.Tensor, w_out: torch.Tensor, gv: torch.Tensor) -> bool:
    """True when ``gemm_swiglu_bwd`` runs as one kernel (``dout`` [M, H], ``w_out`` [I, H], ``gv`` [M, 2 I], bf16)."""
    if not (dout.is_cuda and GEMM_IMPL == "2cta" and _tma_ok(dout, w_out, gv)):
        return False
    I = w_out.shape[0]
    return dout.shape[0] >= 256 and I >= 256 and I % 8 == 0 and gv.shape == (dout.shape[0], 2 * I)


def gemm_swiglu_bwd(dout: torch.Tensor, w_out: torch.Tensor, gv: torch.Tensor) -> torch.Tensor:
    """``d[gate | value]`` [M, 2 I] from ``dout`` [M, H], the down projection ``w_out`` [I, H] and the forward's
    projection ``gv``: the gradient of the activation, ``dout @ w_out^T``, exists only in tensor memory; the GEMM's
    epilogue reads the gate / value tiles and writes the two gradients. Only where ``gemm_swiglu_bwd_fusable``."""
    M, K = dout.shape
    I = w_out.shape[0]
    assert gemm_swiglu_bwd_fusable(dout, w_out, gv)
    dgv = torch.empty_like(gv)
    native.status_tensor()
    _apply_dynamic()
    rc = native.lib().b200_gemm_bf16_2cta_swiglu_bwd(
        native.ptr(dout), native.ptr(w_out), native.ptr(gv), native.ptr(dgv), M, I, K, dout.stride(0), w_out.stride(0),
        gv.stride(0), dgv.stride(0), 0, native.stream_ptr())
    native.check(rc, "b200_gemm_bf16_2cta_swiglu_bwd")
    native.bump()
    return dgv


def gemm_delta_fusable(dout: torch.Tensor, w_o: torch.Tensor, o: torch.Tensor, T: int, head_dim: int) -> bool:
    """True when ``gemm_delta`` runs as one kernel (``dout`` [M, H], ``w_o`` [heads * head_dim, H], ``o`` [M, heads *
    head_dim], bf16; M = batch * T)."""
    if not (dout.is_cuda and GEMM_IMPL == "2cta" and _tma_ok(dout, w_o, o)):
        return False
    N = w_o.shape[0]
    return (head_dim in (64, 128) and N % head_dim == 0 and dout.shape[0] >= 256 and N >= 256 and T > 0
            and dout.shape[0] % T == 0 and o.shape == (dout.shape[0], N))


def gemm_delta(dout: torch.Tensor, w_o: torch.Tensor, o: torch.Tensor, T: int, head_dim: int):
    """Gradient of the attention output and the row sums the attention backward needs, from ONE GEMM:
    ``do = dout @ w_o^T`` [M, heads * head_dim] and ``delta[b, head, t] = sum_d do * o`` (fp32, [batch, heads, T]); the
    epilogue reads the forward's output ``o`` tile by tile. Only where ``gemm_delta_fusable`` holds."""
    M, K = dout.shape
    N = w_o.shape[0]
    assert gemm_delta_fusable(dout, w_o, o, T, head_dim)
    do = torch.empty((M, N), dtype=torch.bfloat16, device=dout.device)
    delta = torch.empty((M // T, N // head_dim, T), dtype=torch.float32, device=dout.device)
    native.status_tensor()
    _apply_dynamic()
    rc = native.lib().b200_gemm_bf16_2cta_delta(
        native.ptr(dout), native.ptr(w_o), native.ptr(do), native.ptr(o), native.ptr(delta), M, N, K, dout.stride(0),
        w_o.stride(0), N, o.stride(0), T, head_dim, _whole_tiles_flag(dout.device), native.stream_ptr())
    native.check(rc, "b200_gemm_bf16_2cta_delta")
    native.bump()
    return do, delta


def gemm_ce_fusable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the LM-head GEMMs with the loss epilogues run for ``x`` [M, K] and ``w`` [V, K] (bf16)."""
    return bool(x.is_cuda and GEMM_IMPL == "2cta" and _tma_ok(x, w) and x.shape[0] >= 256 and w.shape[0] >= 256)


def gemm_ce_stats(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, tlogit: torch.Tensor, col0: int = 0,
                  vocab: int = 0):
    """Logits ``x @ w^T`` that are never stored: returns per-tile row statistics ``(pmax, psum)``, each
    ``[ceil(V / 256), M]`` fp32 (maximum and sum of exp(logit - maximum) over the tile's columns), and writes the
    target's logit of every row whose target lies in ``[col0, col0 + V)`` into ``tlogit`` [M] fp32. ``vocab``
    (size of the whole vocabulary, 0: unknown) lets the bounds-checking build report targets beyond it."""
    M, K = x.shape
    V = w.shape[0]
    assert gemm_ce_fusable(x, w) and targets.dtype == torch.int32 and targets.numel() == M
    nt = (V + 255) // 256
    pmax = torch.empty((nt, M), dtype=torch.float32, device=x.device)
    psum = torch.empty((nt, M), dtype=torch.float32, device=x.device)
    native.status_tensor()
    _apply_dynamic()
    rc = native.lib().b200_gemm_bf16_2cta_ce_stats(
        native.ptr(x), native.ptr(w), M, V, K, x.stride(0), w.stride(0), native.ptr(targets), native.ptr(pmax),
        native.ptr(psum), native.ptr(tlogit), col0, 0, int(vocab), native.stream_ptr())
    native.check(rc, "b200_gemm_bf16_2cta_ce_stats")
    native.bump()
    return pmax, psum


def gemm_ce_dlogits(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, coef: torch.Tensor,
                    col0: int = 0) -> torch.Tensor:
    """``(exp(x @ w^T - lse[row]) - onehot(target)) * coef[row]`` as bf16 [M, V_chunk]: the gradient of the loss
    w.r.t. the logits of vocabulary rows ``col0 .. col0 + V_chunk``, formed in the GEMM epilogue."""
    M, K = x.shape
    C = w.shape[0]
    assert gemm_ce_fusable(x, w) and C % 8 == 0
    out = torch.empty((M, C), dtype=torch.bfloat16, device=x.device)
    native.status_tensor()
    _apply_dynamic()
    rc = native.lib().b200_gemm_bf16_2cta_ce_dlogits(
        native.ptr(x), native.ptr(w), native.ptr(out), M, C, K, x.stride(0), w.stride(0), C, native.ptr(targets),
        native.ptr(lse), native.ptr(coef), col0, native.stream_ptr())
    native.check(rc, "b200_gemm_bf16_2cta_ce_dlogits")
    native.bump()
    return out


def gemm_allgather(a: torch.Tensor, unit_buf: torch.Tensor, b_offset: int, b_shape: tuple, *, trans_b: bool,
                   peer_slices, seg: torch.Tensor, epoch: int, n_copy: int = 8, add: torch.Tensor | None = None,
                   out: torch.Tensor | None = None, trans_a: bool = False, only_b: bool = False) -> torch.Tensor:
    """``out = op(a) @ op(B) (+ add)`` where B is the weight ``b_shape`` stored at element offset
    ``b_offset`` of the local ZeRO unit buffer ``unit_buf`` — and the unit buffer is being filled
    by this same kernel: ``n_copy`` CTAs pull every rank's slice (``peer_slices`` = W device
    pointers, one per rank, same length) over NVLink while the remaining CTAs run the GEMM, each
    waiting only for the rows of B it is about to load. When the kernel finishes the whole unit
    buffer is valid. ``seg`` = this buffer's progress counters (int64 zeros, one per MiB),
    ``epoch`` = 1, 2, ... per use of the buffer. With ``only_b`` the kernel copies just the 32 KiB
    chunks that hold B (``ag_region`` gives their byte range; the caller gathers the rest of the
    unit with ``FusedCollectives.all_gather(..., skip=range)``); ``seg`` must then be zeroed and
    ``epoch`` be 1 for every call, because the range differs from use to use."""
    W = len(peer_slices)
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    if trans_b:
        N, Kb = b_shape
    else:
        Kb, N = b_shape
    if K != Kb:
        raise ValueError(f"gemm_allgather: inner dims differ ({K} vs {Kb})")
    assert a.is_cuda and a.dtype == torch.bfloat16 and unit_buf.dtype == torch.bfloat16
    assert unit_buf.numel() % W == 0
    a, lda = _rowmajor_2d(a)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    flags, ldc = 0, 0
    if add is not None:
        assert add.shape == (M, N) and add.stride(1) == 1 and add.dtype == out.dtype
        ldc = add.stride(0)
        flags |= GEMM_ADD_C
    native.status_tensor()
    src = (ctypes.c_void_p * W)(*[ctypes.c_void_p(int(p)) for p in peer_slices])
    rc = native.lib().b200_gemm_bf16_allgather(
        native.ptr(a), native.ptr(out), native.ptr(add), M, N, K, lda, out.stride(0), ldc, int(trans_a),
        int(not trans_b), flags, ctypes.c_float(1.0), src, native.ptr(unit_buf), native.ptr(seg),
        ctypes.c_ulonglong(unit_buf.numel() // W * 2), ctypes.c_ulonglong(b_offset * 2), W, n_copy,
        ctypes.c_uint(epoch), int(only_b), native.stream_ptr())
    native.check(rc, "b200_gemm_bf16_allgather")
    native.bump()
    return out


def ag_region(slice_bytes: int, world: int, b_offset_bytes: int, b_bytes: int) -> tuple[int, int]:
    """Byte range of the unit buffer that ``gemm_allgather(..., only_b=True)`` fills itself."""
    out = (ctypes.c_ulonglong * 3)()
    native.check(native.lib().b200_ag_region(ctypes.c_ulonglong(slice_bytes), world, ctypes.c_ulonglong(b_offset_bytes),
                                             ctypes.c_ulonglong(b_bytes), out), "ag_region")
    return int(out[0]), int(out[1])


# ---------------------------------------------------------------------------------------------
# Weight-gradient GEMMs on a second stream. Every GEMM here is a persistent kernel that fills the
# GPU, so two of them never run side by side; but on one stream the next kernel cannot start until
# the LAST tile of the previous one has finished, and several training shapes end with a
# part-filled wave (e.g. 2048 x 3072 x 8192 is 1.3 waves of CTA pairs). The weight-gradient GEMMs
# do not feed the activation-gradient chain, so issuing them on a side stream lets their first
# CTAs start on SMs the other kernel has already left.
WGRAD_OVERLAP = True
_wgrad_streams: dict = {}
_wgrad_pending: dict = {}     # device index -> a side-stream GEMM has been issued and not joined yet


def _wgrad_stream(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _wgrad_streams.get(key)
    if st is None:
        st = _wgrad_streams[key] = torch.cuda.Stream(device=device)
    return st


def wgrad_gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a^T @ b`` for a weight gradient; runs on the side stream when overlap is enabled. The
    caller must call ``wgrad_join()`` before the result is consumed on the main stream."""
    if not (WGRAD_OVERLAP and a.is_cuda):
        return gemm(a, b, trans_a=True, out=out)
    cur = torch.cuda.current_stream(a.device)
    ws = _wgrad_stream(a.device)
    ws.wait_stream(cur)
    _wgrad_pending[a.device.index] = True
    with torch.cuda.stream(ws):
        res = gemm(a, b, trans_a=True, out=out)
    a.record_stream(ws)
    b.record_stream(ws)
    return res


def wgrad_event(device):
    """An event after everything issued so far on the weight-gradient side stream of ``device`` (None when
    that stream has never been used): what a consumer on a third stream waits for instead of joining."""
    dev = torch.device(device)
    if not WGRAD_OVERLAP or dev.type != "cuda":
        return None
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    ws = _wgrad_streams.get(key)
    if ws is None:
        return None
    ev = torch.cuda.Event()
    ev.record(ws)
    return ev


def wgrad_join(device=None) -> None:
    if not WGRAD_OVERLAP or not torch.cuda.is_available():
        return
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type != "cuda":
        return
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    ws = _wgrad_streams.get(key)
    if ws is not None:
        torch.cuda.current_stream(dev).wait_stream(ws)
    _wgrad_pending[key] = False
