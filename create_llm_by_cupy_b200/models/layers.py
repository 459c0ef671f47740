"""Transformer layers with hand-written forward / backward (no autograd).

Each layer follows the protocol of the reference (``params`` list, ``grads`` list filled by
``backward``, ``forward``/``backward`` methods; model/fast_layers.py:75-584, 681-824, 834-1276,
1280-1488, 1494-1512) but is built for a 180 GB part: by default every intermediate that
backward needs is kept instead of recomputed, residual adds are fused into the projection GEMM
epilogues, the rotary embedding is fused into the attention kernels, and weight gradients are
written by the GEMM straight into views of the flat gradient bucket the ZeRO manager hands in
(``grad_out``), so no concatenate / copy pass exists. The recompute switches of the reference
(``gqa_cache_out_value``, ``swiglu_cache_gate``) are still honoured when set to False.

Tensors are ``[M, H]`` with ``M = B*T`` tokens, bf16 on CUDA (fp32 on the CPU path).
"""
from __future__ import annotations

import math

import torch

from ..ops import functional as F


def init_weight(shape, std: float, dtype, device, generator=None) -> torch.Tensor:
    """N(0, std) initialiser (model/functions.py:62-63), drawn in fp32 then cast."""
    w = torch.randn(*shape, dtype=torch.float32, device=generator.device if generator is not None else device,
                    generator=generator) * std
    return w.to(device=device, dtype=dtype)


def _weight_gemm(layer, a: torch.Tensor, widx: int, *, trans_b: bool = False, add=None) -> torch.Tensor:
    """``a @ W`` (or ``a @ W^T``) for ``W = layer.params[widx]``. When the ZeRO manager deferred the
    all-gather of this layer's unit, this GEMM is the one that carries it: the fused kernel pulls
    the unit from the peers while it multiplies (``pending_gather`` is set by the manager and names
    each parameter by its index in ``model.params``)."""
    pg = getattr(layer, "pending_gather", None)
    if pg is not None:
        layer.pending_gather = None
        idx = layer._zero3_param_indices[widx]
        if not pg.done and pg.mgr.layout.slots[idx].unit == pg.uid and a.is_cuda:
            out = pg.gemm(a, idx, trans_b=trans_b, add=add)
            pg.mgr.deferred.pop(pg.uid, None)
            return out
        pg.flush()
        pg.mgr.deferred.pop(pg.uid, None)
    return F.gemm(a, layer.params[widx], trans_b=trans_b, add=add)


def _store_grad(dst: torch.Tensor | None, src: torch.Tensor) -> torch.Tensor:
    if dst is None:
        return src
    if dst.data_ptr() != src.data_ptr():
        dst.copy_(src)
    return dst


class RMSNorm:
    """y = x * rsqrt(mean(x^2) + eps) * gamma. Keeps its input and the per-row rsqrt."""

    def __init__(self, hidden_size: int, dtype=torch.bfloat16, device="cpu", eps: float = 1e-6):
        self.hidden_size = hidden_size
        self.eps = eps
        self.params = [torch.ones(hidden_size, dtype=dtype, device=device)]
        self.grads = [None]
        self.cache = None

    def forward(self, x: torch.Tensor, train_flg: bool = True) -> torch.Tensor:
        y, rstd = F.rmsnorm_fwd(x, self.params[0], self.eps)
        self.cache = (x, rstd) if train_flg else None
        return y

    def backward(self, dy: torch.Tensor, add: torch.Tensor | None = None, grad_out=None) -> torch.Tensor:
        """Returns dx (+ ``add``, the gradient that bypasses the norm through the residual)."""
        x, rstd = self.cache
        dx, dgamma = F.rmsnorm_bwd(dy, x, self.params[0], rstd, add=add)
        self.grads = [_store_grad(grad_out[0] if grad_out else None, dgamma)]
        self.cache = None
        return dx


class GroupedQueryAttention:
    """Fused [K|Q|V] projection, causal GQA flash attention with in-kernel RoPE, output projection.

    params: ``W_KQV [H, KVH*D + H + KVH*D]`` (column order K, Q, V) and ``W_O [H, H]``, both
    ``[in, out]`` as in the reference (model/fast_layers.py:101-105).
    """

    def __init__(self, hidden_size, time_size, q_head, kv_head, layer_num, dropout_rate=0.0,
                 dtype=torch.bfloat16, device="cpu", generator=None, init_std=None, rope_base=10000.0):
        assert hidden_size % q_head == 0 and q_head % kv_head == 0
        self.H, self.T = hidden_size, time_size
        self.QH, self.KVH = q_head, kv_head
        self.D = hidden_size // q_head
        self.KV = kv_head * self.D
        self.scale = 1.0 / math.sqrt(self.D)
        self.rope_base = rope_base
        self.dropout_rate = dropout_rate
        std_in = init_std if init_std is not None else 1.0 / math.sqrt(hidden_size)
        std_out = init_std if init_std is not None else 1.0 / math.sqrt(2.0 * hidden_size * layer_num)
        self.params = [
            init_weight((hidden_size, self.KV + hidden_size + self.KV), std_in, dtype, device, generator),
            init_weight((hidden_size, hidden_size), std_out, dtype, device, generator),
        ]
        self.grads = [None, None]
        self.cache = None
        self.cache_out_value = True      # keep the attention output for dW_O (else recompute flash fwd)
        self.cache_kqv = True            # keep the projection (else re-project from x in backward)
        self.cache_attn = False          # dense path only: keep the [B,QH,T,T] probabilities
        self.flash_backend = "b200"      # "none" selects the dense verification path
        # Two dropouts as in the reference (model/fast_layers.py:93-95, 316, 346), only built when
        # dropout_rate != 0: on the attention probabilities - which forces the dense attention path while
        # training, there is no dropout inside the flash kernels - and on the projected output.
        self.drop_attn = TimeDropout(dropout_rate, dtype, generator) if dropout_rate else None
        self.drop = TimeDropout(dropout_rate, dtype, generator) if dropout_rate else None
        self._dense = False              # the pass in flight runs the dense attention path

    # -- helpers ---------------------------------------------------------------------------
    def _split(self, kqv: torch.Tensor, B: int, T: int):
        v3 = kqv.view(B, T, -1)
        k = v3[:, :, :self.KV].unflatten(2, (self.KVH, self.D))
        q = v3[:, :, self.KV:self.KV + self.H].unflatten(2, (self.QH, self.D))
        v = v3[:, :, self.KV + self.H:].unflatten(2, (self.KVH, self.D))
        return q, k, v

    def _rope(self, T, device):
        return F.rope_table(max(T, self.T), self.D, self.rope_base, device)

    def _prerotate(self, x) -> bool:
        """head_dim 128 (and the forward of head_dim 64) on CUDA runs the tcgen05 attention kernels, which
        take Q and K already rotated: the rotary embedding is then applied in place to the [K|Q] columns of
        the packed projection (one pass over 5/6 of it) and undone on d[K|Q] in the epilogues of the
        backward kernels (head_dim 128) or by a pass after them."""
        return x.is_cuda and not self._dense and F.flash_tc_forward_dim(self.D)

    def _project(self, x, T, tabs, first: bool):
        """K | Q | V projection; on the pre-rotating path K and Q leave it rotated - inside the GEMM's epilogue
        where that form exists, else by an in-place pass over the [K|Q] columns."""
        pre = self._prerotate(x)
        rope_cols = (self.KVH + self.QH) * self.D
        if (pre and getattr(self, "pending_gather", None) is None
                and F.gemm_rope_fusable(x, self.params[0], self.D, rope_cols)):
            return F.gemm_rope(x, self.params[0], tabs[0], tabs[1], T, self.D, rope_cols)
        kqv = _weight_gemm(self, x, 0) if first else F.gemm(x, self.params[0])
        if pre:
            F.rope_inplace(kqv, tabs[0], tabs[1], T, self.KVH + self.QH, self.D, col0=0)
        return kqv

    def _attend(self, q, k, v, valid_len, tabs, train_flg: bool = False):
        if self._dense:
            o, lse, p, _, _ = F._attn_reference(q, k, v, valid_len, self.scale, tabs[0], tabs[1])
            if self.drop_attn is not None and train_flg:
                vx = v.float().repeat_interleave(self.QH // self.KVH, dim=2)
                o = torch.einsum("bhts,bshd->bthd", self.drop_attn.forward(p, True), vx)
            return o.to(q.dtype).contiguous(), lse
        if self._prerotate(q):
            return F.flash_attn_fwd(q, k, v, valid_len=valid_len, scale=self.scale, rope=None)
        return F.flash_attn_fwd(q, k, v, valid_len=valid_len, scale=self.scale, rope=tabs)

    # -- training path ---------------------------------------------------------------------
    def forward(self, x: torch.Tensor, B: int, T: int, valid_len=None, residual=None,
                train_flg: bool = True) -> torch.Tensor:
        """x: normed input [M, H]. Returns W_O(attn) (+ residual) as [M, H]."""
        tabs = self._rope(T, x.device)
        self._dense = self.flash_backend == "none" or (self.drop_attn is not None and train_flg)
        kqv = self._project(x, T, tabs, True)
        q, k, v = self._split(kqv, B, T)
        o, lse = self._attend(q, k, v, valid_len, tabs, train_flg)
        if self.drop is not None and train_flg:
            out = self.drop.forward(F.gemm(o.view(B * T, self.H), self.params[1]), True)
            out = F.add(out, residual) if residual is not None else out
        else:
            out = F.gemm(o.view(B * T, self.H), self.params[1], add=residual)
        if train_flg:
            self.cache = (x, B, T, valid_len, kqv if self.cache_kqv else None,
                          o if self.cache_out_value else None, lse)
        else:
            self.cache = None
        return out

    def backward(self, dout: torch.Tensor, grad_out=None) -> torch.Tensor:
        x, B, T, valid_len, kqv, o, lse = self.cache
        if self.drop is not None:
            dout = self.drop.backward(dout)
        tabs = self._rope(T, x.device)
        if kqv is None:
            kqv = self._project(x, T, tabs, False)
        q, k, v = self._split(kqv, B, T)
        if o is None:
            if self._dense and self.drop_attn is not None:
                raise RuntimeError("gqa_cache_out_value=False cannot be combined with attention dropout: the "
                                   "recomputed forward would draw a new mask")
            o, lse = self._attend(q, k, v, valid_len, tabs)
        go = grad_out if grad_out else (None, None)
        dW_O = F.wgrad_gemm(o.view(B * T, self.H), dout, out=go[1])
        delta = None
        o2d = o.view(B * T, self.H)
        if (F.DELTA_EPILOGUE and not self._dense and self._prerotate(x)
                and F.gemm_delta_fusable(dout, self.params[1], o2d, T, self.D)):
            # d(attention output) and the backward's row sums sum_d dO * O from one GEMM
            do, delta = F.gemm_delta(dout, self.params[1], o2d, T, self.D)
        else:
            do = F.gemm(dout, self.params[1], trans_b=True)
        dkqv = torch.empty_like(kqv)
        dq, dk, dv = self._split(dkqv, B, T)
        if self._dense:
            # dense path (verification, or training with attention dropout): the fp32 restatement, on the
            # device the tensors live on
            F._attn_bwd_reference(do.view(B, T, self.QH, self.D), q, k, v, o, valid_len, self.scale, tabs[0], tabs[1],
                                  out=(dq, dk, dv), p_drop=self.drop_attn)
        elif self._prerotate(x):
            fused = F.flash_bwd_can_unrotate(q)          # inverse RoPE in the kernels' epilogues
            F.flash_attn_bwd(do.view(B, T, self.QH, self.D), q, k, v, o, lse, valid_len=valid_len,
                             scale=self.scale, rope=None, out=(dq, dk, dv), unrotate=tabs if fused else None,
                             delta=delta)
            if not fused:
                F.rope_inplace(dkqv, tabs[0], tabs[1], T, self.KVH + self.QH, self.D, col0=0, inverse=True)
        else:
            F.flash_attn_bwd(do.view(B, T, self.QH, self.D), q, k, v, o, lse, valid_len=valid_len,
                             scale=self.scale, rope=tabs, out=(dq, dk, dv))
        dW_KQV = F.wgrad_gemm(x, dkqv, out=go[0])
        dx = F.gemm(dkqv, self.params[0], trans_b=True)
        self.grads = [dW_KQV, dW_O]
        self.cache = None
        return dx

    # -- incremental decoding --------------------------------------------------------------
    def prefill(self, x, B, T, kcache, vcache, residual=None):
        """Full-sequence forward that also fills the KV cache [B, KVH, Tmax, D] (K stored rotated)."""
        kqv = F.gemm(x, self.params[0])
        tabs = self._rope(kcache.shape[2], x.device)
        F.rope_inplace(kqv, tabs[0], tabs[1], T, self.KVH, self.D, col0=0)
        F.rope_inplace(kqv, tabs[0], tabs[1], T, self.QH, self.D, col0=self.KV)
        q, k, v = self._split(kqv, B, T)
        kcache[:, :, :T].copy_(k.permute(0, 2, 1, 3))
        vcache[:, :, :T].copy_(v.permute(0, 2, 1, 3))
        if self.flash_backend == "none":
            o, _, _, _, _ = F._attn_reference(q, k, v, None, self.scale, None, None)
            o = o.to(x.dtype).contiguous()
        else:
            o, _ = F.flash_attn_fwd(q, k, v, scale=self.scale, rope=None)
        return F.gemm(o.reshape(B * T, self.H), self.params[1], add=residual)

    def decode_step(self, x, pos: int, kcache, vcache, lens, residual=None):
        """x: [B, H] normed hidden state of the token at position ``pos`` (same for the batch)."""
        B = x.shape[0]
        kqv = F.gemm(x, self.params[0])
        tabs = self._rope(kcache.shape[2], x.device)
        F.rope_inplace(kqv, tabs[0], tabs[1], 1, self.KVH, self.D, col0=0, pos0=pos)
        F.rope_inplace(kqv, tabs[0], tabs[1], 1, self.QH, self.D, col0=self.KV, pos0=pos)
        k = kqv[:, :self.KV].view(B, self.KVH, self.D)
        q = kqv[:, self.KV:self.KV + self.H].reshape(B, self.QH, self.D)
        v = kqv[:, self.KV + self.H:].view(B, self.KVH, self.D)
        kcache[:, :, pos].copy_(k)
        vcache[:, :, pos].copy_(v)
        o = F.decode_attn(q.contiguous(), kcache, vcache, lens, self.scale)
        return F.gemm(o.view(B, self.H), self.params[1], add=residual)

    @staticmethod
    def convert_legacy_weights(W_K, W_Q, W_V, W_O):
        """Separate projections ([H, KV], [H, H], [H, KV], [H, H]) -> fused [W_KQV, W_O]
        (the job of model/fast_layers.py:566-584)."""
        return [torch.cat([W_K, W_Q, W_V], dim=1).contiguous(), W_O]


class SwiGLU:
    """``(silu(x W_gate) * (x W_value)) W_out`` with the fused ``W_gate_val = [gate | value]``.

    The inner size defaults to ``int(8H/3)`` as in the reference (model/fast_layers.py:710) and
    can be set explicitly with ``ffn_size``.
    """

    def __init__(self, hidden_size, layer_num, dtype=torch.bfloat16, dropout_rate=0.0, device="cpu",
                 generator=None, ffn_size=None, init_std=None):
        self.H = hidden_size
        self.I = int(ffn_size) if ffn_size else int(hidden_size * 8 / 3)
        std_in = init_std if init_std is not None else 1.0 / math.sqrt(hidden_size)
        std_out = init_std if init_std is not None else 1.0 / math.sqrt(2.0 * layer_num * self.I)
        self.params = [
            init_weight((hidden_size, 2 * self.I), std_in, dtype, device, generator),
            init_weight((self.I, hidden_size), std_out, dtype, device, generator),
        ]
        self.grads = [None, None]
        self.cache = None
        self.cache_gate = True
        self.dropout_rate = dropout_rate
        self.drop = TimeDropout(dropout_rate, dtype, generator) if dropout_rate else None

    def _gate_act(self, x: torch.Tensor, keep_gv: bool):
        """(gv or None, act): the gate|value projection with the activation applied in the GEMM's epilogue
        where that form exists (one kernel, the projection is only written when the backward will read it),
        else the GEMM followed by the activation kernel."""
        if (F.SWIGLU_EPILOGUE and getattr(self, "pending_gather", None) is None
                and F.gemm_swiglu_fusable(x, self.params[0])):
            return F.gemm_swiglu(x, self.params[0], keep_gv=keep_gv)
        gv = _weight_gemm(self, x, 0)
        return gv, F.swiglu_fwd(gv)

    def forward(self, x: torch.Tensor, residual=None, train_flg: bool = True) -> torch.Tensor:
        keep = train_flg and self.cache_gate
        gv, act = self._gate_act(x, keep)
        if self.drop is not None and train_flg:
            out = self.drop.forward(F.gemm(act, self.params[1]), True)
            out = F.add(out, residual) if residual is not None else out
        else:
            out = F.gemm(act, self.params[1], add=residual)
        self.cache = (x, gv if keep else None, act if keep else None) if train_flg else None
        return out

    def backward(self, dout: torch.Tensor, grad_out=None) -> torch.Tensor:
        x, gv, act = self.cache
        if self.drop is not None:
            dout = self.drop.backward(dout)
        if gv is None:
            gv, act = self._gate_act(x, True)
        go = grad_out if grad_out else (None, None)
        dW_out = F.wgrad_gemm(act, dout, out=go[1])
        if (F.SWIGLU_EPILOGUE and getattr(self, "pending_gather", None) is None
                and F.gemm_swiglu_bwd_fusable(dout, self.params[1], gv)):
            dgv = F.gemm_swiglu_bwd(dout, self.params[1], gv)      # d(act) never leaves tensor memory
        else:
            dact = _weight_gemm(self, dout, 1, trans_b=True)
            dgv = F.swiglu_bwd(dact, gv)
        dW_gv = F.wgrad_gemm(x, dgv, out=go[0])
        dx = F.gemm(dgv, self.params[0], trans_b=True)
        self.grads = [dW_gv, dW_out]
        self.cache = None
        return dx


class TimeEmbedding_shard:
    """Token embedding lookup on a gathered ``[V, H]`` table; the pad id maps to a zero row
    (model/fast_layers.py:1494-1512 zeroes that row of the table; here the gather does it)."""

    def __init__(self, padding_id: int, dtype=torch.bfloat16):
        self.padding_id = padding_id
        self.idx = None

    def forward(self, W: torch.Tensor, idx: torch.Tensor, train_flg: bool = True) -> torch.Tensor:
        flat = idx.reshape(-1).to(torch.int32)
        self.idx = flat if train_flg else None
        return F.embedding_fwd(W, flat, self.padding_id)

    def backward(self, dW: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
        """dW[idx] += dout (dW already holds the LM-head gradient when the table is tied)."""
        F.embedding_bwd(dW, self.idx, dout, self.padding_id)
        self.idx = None
        return dW


class ChunkedCrossEntropy_Share:
    """LM head + mean cross-entropy over non-pad targets without an ``[M, V]`` tensor
    (reference: model/fast_layers.py:1280-1488, which makes two chunked passes forward and one backward).

    On CUDA the logits never reach memory. Forward: ONE GEMM over the whole vocabulary whose epilogue folds
    each 256-column tile of the fp32 accumulator into per-row (max, sum-exp, target logit); a small merge gives
    the row's log-sum-exp. Backward walks the vocabulary in chunks of ``chunk_size``: the logits of a chunk are
    recomputed by a GEMM whose epilogue turns them into ``(softmax - onehot) * GradScale / n_valid`` in bf16 (the
    only [M, chunk] tensor that exists), which feeds the two gradient GEMMs; ``dW`` rows go to
    ``grad_writer(row_start, row_end)`` -> destination view, so they land directly in the gradient bucket.

    Where the fused GEMMs do not apply (CPU tensors, tiny shapes, ``cache_logits`` asked for explicitly) the
    chunked form with fp32 logits per chunk is used: one pass forward, logits kept for the backward only when
    ``cache_logits``.
    """

    def __init__(self, padding_id: int, chunk_size: int = 8192, dtype=torch.bfloat16, cache_logits: bool = False):
        self.padding_id = padding_id
        self.chunk_size = int(chunk_size)
        self.cache_logits = cache_logits
        self.cache = None

    def _chunks(self, V: int):
        c = self.chunk_size if self.chunk_size > 0 else V
        return [(s, min(s + c, V)) for s in range(0, V, c)]

    def _fused(self, x: torch.Tensor, W: torch.Tensor) -> bool:
        return bool(F.CE_EPILOGUE and not self.cache_logits and F.gemm_ce_fusable(x, W))

    def forward(self, x: torch.Tensor, t: torch.Tensor, W: torch.Tensor, train_flg: bool = True) -> torch.Tensor:
        """x [M, H], t [M] int32 targets, W [V, H]. Returns the scalar mean loss (device tensor)."""
        M = x.shape[0]
        t = t.reshape(-1).to(torch.int32)
        tlogit = torch.zeros(M, dtype=torch.float32, device=x.device)
        kept = None
        if self._fused(x, W):
            pmax, psum = F.gemm_ce_stats(x, W, t, tlogit, vocab=W.shape[0])
            rmax, rsum = F.ce_merge(pmax, psum)
        else:
            rmax = torch.empty(M, dtype=torch.float32, device=x.device)
            rsum = torch.empty_like(rmax)
            kept = [] if (train_flg and self.cache_logits) else None
            for i, (s, e) in enumerate(self._chunks(W.shape[0])):
                logits = F.gemm(x, W[s:e], trans_b=True, out_dtype=torch.float32)
                F.ce_stats(logits, t, rmax, rsum, tlogit, s, i == 0)
                if kept is not None:
                    kept.append(logits)
        loss_cnt = F.ce_loss(rmax, rsum, tlogit, t, self.padding_id)
        if train_flg:
            self.cache = (x, t, rmax, rsum, loss_cnt, kept)
        self.loss_cnt = loss_cnt
        return loss_cnt[0] / loss_cnt[1].clamp_min(1.0)

    def backward(self, W: torch.Tensor, GradScale: float = 1.0, grad_writer=None) -> torch.Tensor:
        """Returns dx [M, H]. ``grad_writer(s, e)`` must return the [e-s, H] view that receives
        dW[s:e] (overwritten); without it the chunks are collected in ``self.dW``."""
        x, t, rmax, rsum, loss_cnt, kept = self.cache
        dx = None
        self.dW = None
        if grad_writer is None:
            self.dW = torch.empty_like(W)
        fused = kept is None and self._fused(x, W)
        if fused:
            lse, coef = F.ce_row_coef(rmax, rsum, t, loss_cnt, self.padding_id, float(GradScale))
        for i, (s, e) in enumerate(self._chunks(W.shape[0])):
            if fused and (e - s) % 8 == 0 and e - s >= 256:
                dlog = F.gemm_ce_dlogits(x, W[s:e], t, lse, coef, col0=s)
            else:
                logits = kept[i] if kept is not None else F.gemm(x, W[s:e], trans_b=True, out_dtype=torch.float32)
                dlog = F.ce_dlogits(logits, t, rmax, rsum, loss_cnt, s, self.padding_id, float(GradScale), x.dtype)
                if kept is not None:
                    kept[i] = None
            dst = grad_writer(s, e) if grad_writer is not None else self.dW[s:e]
            F.gemm(dlog, x, trans_a=True, out=dst)
            dx = F.gemm(dlog, W[s:e], out=dx, add=dx) if dx is not None else F.gemm(dlog, W[s:e])
        self.cache = None
        return dx


class TimeDropout:
    """Inverted dropout whose mask is kept as packed bits, one bit per element
    (model/fast_layers.py:616-673). The keep pattern is a counter-based function of (seed, running element
    offset), identical on CPU and GPU. The seed is derived from the model generator's initial seed and the
    layer's construction index; it does not draw from the generator, so a model with dropout starts from
    the same weights as one without. Only built when ``dropout_rate != 0``; the benchmark configurations use 0."""

    _built = 0

    def __init__(self, dropout_rate: float, dtype=torch.bfloat16, generator=None):
        self.p = float(dropout_rate)
        self.mask = None            # uint8 [(n + 7) / 8]
        self.mask_shape = None
        base = generator.initial_seed() if generator is not None else 0
        TimeDropout._built += 1
        self.seed = (base * 0x9E3779B97F4A7C15 + TimeDropout._built * 0xD1B54A32D192ED03) & ((1 << 62) - 1)
        self.offset = 0

    def forward(self, x: torch.Tensor, train_flg: bool = True) -> torch.Tensor:
        if not train_flg or self.p <= 0.0:
            self.mask = None
            return x
        out, self.mask = F.dropout_fwd(x, self.p, self.seed, self.offset)
        self.mask_shape = tuple(x.shape)
        self.offset += (x.numel() + 7) // 8 * 8
        return out

    def reapply(self, x: torch.Tensor) -> torch.Tensor:
        """x * keep / (1 - p) with the mask of the last forward (kept for ``backward``)."""
        return x if self.mask is None else F.dropout_bwd(x, self.mask, self.p)

    def backward(self, dout: torch.Tensor) -> torch.Tensor:
        if self.mask is None:
            return dout
        out = F.dropout_bwd(dout, self.mask, self.p)
        self.mask = None
        self.mask_shape = None
        return out


class SoftMax:
    """fp32 softmax layer with its backward (model/fast_layers.py:590-612); kept for parity."""

    def __init__(self):
        self.out = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self.out = torch.softmax(x.float(), dim=-1)
        return self.out.to(x.dtype)

    def backward(self, dout: torch.Tensor) -> torch.Tensor:
        y = self.out
        d = dout.float()
        return (y * (d - (d * y).sum(-1, keepdim=True))).to(dout.dtype)
