"""NumPy (float64) oracle of the whole model: forward loss, analytic backward, AdamW step and
greedy decoding. It is the independent restatement every other path (torch CPU layers, CUDA
kernels, sharded managers) is tested against, and the CPU configuration of the benchmark suite.

The math follows the reference's layers (model/fast_layers.py, model/flash_attention.py:51-176,
model/optimizer.py:55-99) written densely: no tiling, no chunking, no mixed precision.
Parameters are taken in ``Cupa_ver4.params`` order.
"""
from __future__ import annotations

import math

import numpy as np


class OracleConfig:
    def __init__(self, vocab, hidden, layers, q_head, kv_head, ffn, pad_id, tied=True, rope_base=10000.0,
                 eps=1e-6):
        self.V, self.H, self.L = vocab, hidden, layers
        self.QH, self.KVH = q_head, kv_head
        self.D = hidden // q_head
        self.I = ffn
        self.pad = pad_id
        self.tied = tied
        self.rope_base = rope_base
        self.eps = eps

    @classmethod
    def from_model_dic(cls, d):
        H = d["hidden_size"]
        return cls(d["vocab_size"], H, d["layer_num"], d["q_head"], d["kv_head"],
                   int(d["ffn_size"]) if d.get("ffn_size") else int(H * 8 / 3),
                   d["padding_id"] if d.get("padding_id") is not None else -1,
                   bool(d.get("tie_embeddings", True)), float(d.get("rope_base", 10000.0)))


def _rope_tables(T, D, base):
    j = np.arange(D // 2, dtype=np.float64)
    freq = base ** (-2.0 * j / D)
    ang = np.arange(T, dtype=np.float64)[:, None] * freq[None, :]
    return np.cos(ang), np.sin(ang)


def _rope(x, cos, sin):
    """x [B, T, heads, D]; half-split pairing."""
    D = x.shape[-1]
    x1, x2 = x[..., :D // 2], x[..., D // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def _rope_t(dy, cos, sin):
    D = dy.shape[-1]
    y1, y2 = dy[..., :D // 2], dy[..., D // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return np.concatenate([y1 * c + y2 * s, y2 * c - y1 * s], -1)


def _rms_fwd(x, g, eps):
    r = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return x * r * g, r


def _rms_bwd(dy, x, g, r):
    xh = x * r
    wdy = dy * g
    dx = r * (wdy - xh * (wdy * xh).mean(-1, keepdims=True))
    return dx, (dy * xh).reshape(-1, x.shape[-1]).sum(0)


def _silu(x):
    return x / (1.0 + np.exp(-x))


class Oracle:
    def __init__(self, cfg: OracleConfig, params):
        self.c = cfg
        self.p = [np.asarray(p, dtype=np.float64).copy() for p in params]

    # parameter accessors -------------------------------------------------------------------
    def block(self, b):
        return self.p[b * 6:(b + 1) * 6]

    @property
    def emb(self):
        return self.p[self.c.L * 6]

    @property
    def head(self):
        return self.p[self.c.L * 6 + (0 if self.c.tied else 1)]

    @property
    def gfinal(self):
        return self.p[-1]

    # forward ---------------------------------------------------------------------------------
    def forward(self, x, t, valid_len=None, keep=True):
        c = self.c
        B, T = x.shape
        cos, sin = _rope_tables(T, c.D, c.rope_base)
        emb = self.emb
        h = emb[np.clip(x, 0, None)] * (x != c.pad)[..., None]
        R = c.QH // c.KVH
        KV = c.KVH * c.D
        mask = np.tril(np.ones((T, T), dtype=bool))[None, None]
        if valid_len is not None:
            mask = mask & (np.arange(T)[None, :] < np.asarray(valid_len)[:, None])[:, None, None, :]
        saved = []
        for b in range(c.L):
            Wkqv, Wo, Wgv, Wout, g1, g2 = self.block(b)
            n1, r1 = _rms_fwd(h, g1, c.eps)
            kqv = n1 @ Wkqv
            k = kqv[..., :KV].reshape(B, T, c.KVH, c.D)
            q = kqv[..., KV:KV + c.H].reshape(B, T, c.QH, c.D)
            v = kqv[..., KV + c.H:].reshape(B, T, c.KVH, c.D)
            qr, kr = _rope(q, cos, sin), _rope(k, cos, sin)
            kx, vx = np.repeat(kr, R, axis=2), np.repeat(v, R, axis=2)
            s = np.einsum("bthd,bshd->bhts", qr, kx) / math.sqrt(c.D)
            s = np.where(mask, s, -np.inf)
            s = s - s.max(-1, keepdims=True)
            pr = np.exp(s)
            pr = pr / pr.sum(-1, keepdims=True)
            o = np.einsum("bhts,bshd->bthd", pr, vx).reshape(B, T, c.H)
            h2 = h + o @ Wo
            n2, r2 = _rms_fwd(h2, g2, c.eps)
            gv = n2 @ Wgv
            gate, val = gv[..., :c.I], gv[..., c.I:]
            act = _silu(gate) * val
            h3 = h2 + act @ Wout
            if keep:
                saved.append((h, n1, r1, qr, kr, v, pr, o, h2, n2, r2, gate, val, act))
            h = h3
        nf, rf = _rms_fwd(h, self.gfinal, c.eps)
        logits = nf @ self.head.T
        m = logits.max(-1, keepdims=True)
        lse = m[..., 0] + np.log(np.exp(logits - m).sum(-1))
        valid = (t != c.pad)
        tl = np.take_along_axis(logits, np.clip(t, 0, None)[..., None], -1)[..., 0]
        n_valid = max(valid.sum(), 1)
        loss = ((lse - tl) * valid).sum() / n_valid
        if keep:
            self._saved = (x, t, saved, h, nf, rf, logits, lse, valid, n_valid, cos, sin, mask)
        return float(loss)

    def logits(self, x):
        self.forward(x, np.zeros_like(x), keep=True)
        return self._saved[6]

    # backward --------------------------------------------------------------------------------
    def backward(self, grad_scale=1.0):
        """Gradients of ``grad_scale * loss`` in ``params`` order."""
        c = self.c
        x, t, saved, hL, nf, rf, logits, lse, valid, n_valid, cos, sin, mask = self._saved
        B, T = x.shape
        R = c.QH // c.KVH
        KV = c.KVH * c.D
        grads = [np.zeros_like(p) for p in self.p]
        prob = np.exp(logits - lse[..., None])
        dlog = prob
        np.put_along_axis(dlog, np.clip(t, 0, None)[..., None],
                          np.take_along_axis(dlog, np.clip(t, 0, None)[..., None], -1) - 1.0, -1)
        dlog = dlog * (valid[..., None] * grad_scale / n_valid)
        head_idx = c.L * 6 + (0 if c.tied else 1)
        grads[head_idx] += dlog.reshape(-1, c.V).T @ nf.reshape(-1, c.H)
        dnf = dlog @ self.head
        dh, dg = _rms_bwd(dnf, hL, self.gfinal, rf)
        grads[-1] += dg
        for b in range(c.L - 1, -1, -1):
            Wkqv, Wo, Wgv, Wout, g1, g2 = self.block(b)
            h, n1, r1, qr, kr, v, pr, o, h2, n2, r2, gate, val, act = saved[b]
            base = b * 6
            grads[base + 3] += act.reshape(-1, c.I).T @ dh.reshape(-1, c.H)
            dact = dh @ Wout.T
            sg = 1.0 / (1.0 + np.exp(-gate))
            dgate = dact * val * sg * (1.0 + gate * (1.0 - sg))
            dval = dact * gate * sg
            dgv = np.concatenate([dgate, dval], -1)
            grads[base + 2] += n2.reshape(-1, c.H).T @ dgv.reshape(-1, 2 * c.I)
            dn2 = dgv @ Wgv.T
            dx2, dg2 = _rms_bwd(dn2, h2, g2, r2)
            grads[base + 5] += dg2
            dh2 = dh + dx2
            grads[base + 1] += o.reshape(-1, c.H).T @ dh2.reshape(-1, c.H)
            do = (dh2 @ Wo.T).reshape(B, T, c.QH, c.D)
            kx, vx = np.repeat(kr, R, axis=2), np.repeat(v, R, axis=2)
            dvx = np.einsum("bhts,bthd->bshd", pr, do)
            dp = np.einsum("bthd,bshd->bhts", do, vx)
            ds = pr * (dp - (dp * pr).sum(-1, keepdims=True)) / math.sqrt(c.D)
            dqr = np.einsum("bhts,bshd->bthd", ds, kx)
            dkx = np.einsum("bhts,bthd->bshd", ds, qr)
            dkr = dkx.reshape(B, T, c.KVH, R, c.D).sum(3)
            dv = dvx.reshape(B, T, c.KVH, R, c.D).sum(3)
            dq, dk = _rope_t(dqr, cos, sin), _rope_t(dkr, cos, sin)
            dkqv = np.concatenate([dk.reshape(B, T, KV), dq.reshape(B, T, c.H), dv.reshape(B, T, KV)], -1)
            grads[base + 0] += n1.reshape(-1, c.H).T @ dkqv.reshape(-1, KV * 2 + c.H)
            dn1 = dkqv @ Wkqv.T
            dx1, dg1 = _rms_bwd(dn1, h, g1, r1)
            grads[base + 4] += dg1
            dh = dh2 + dx1
        emb_idx = c.L * 6
        keep = (x != c.pad)
        np.add.at(grads[emb_idx], x[keep], dh[keep])
        return grads

    # optimizer ---------------------------------------------------------------------------------
    def init_adam(self):
        self.m = [np.zeros_like(p) for p in self.p]
        self.v = [np.zeros_like(p) for p in self.p]
        self.t = 0

    def adam_step(self, grads, lr, beta1=0.9, beta2=0.99, eps=1e-6, wd=0.1, max_grad_norm=0.0):
        """AdamW as model/optimizer.py:69-99: decoupled decay on every parameter, bias-corrected
        m and v; optional global-norm clip min(1, max/(norm + 1e-6)) (model/ZeRO3.py:358-360)."""
        self.t += 1
        if max_grad_norm > 0:
            norm = math.sqrt(sum(float((g * g).sum()) for g in grads))
            coef = min(1.0, max_grad_norm / (norm + 1e-6))
            grads = [g * coef for g in grads]
        mc = 1.0 / (1.0 - beta1 ** self.t)
        vc = 1.0 / (1.0 - beta2 ** self.t)
        for i, g in enumerate(grads):
            self.m[i] = beta1 * self.m[i] + (1 - beta1) * g
            self.v[i] = beta2 * self.v[i] + (1 - beta2) * g * g
            if wd > 0:
                self.p[i] *= (1.0 - lr * wd)
            self.p[i] -= lr * (self.m[i] * mc) / (np.sqrt(self.v[i] * vc) + eps)

    # decoding ----------------------------------------------------------------------------------
    def greedy(self, prompt, n_new):
        toks = list(prompt)
        for _ in range(n_new):
            x = np.asarray(toks, dtype=np.int64)[None, :]
            lg = self.logits(x)[0, -1].copy()
            if 0 <= self.c.pad < self.c.V:
                lg[self.c.pad] = -np.inf
            toks.append(int(lg.argmax()))
        return toks[len(prompt):]


def cosine_lr(step: int, lr_max: float, lr_mini: float, warm_up: int, total_steps: int) -> float:
    """Linear warm-up then cosine decay (model/optimizer.py:55-62); ``step`` counts from 1."""
    if step < warm_up:
        return lr_max * step / warm_up
    progress = (step - warm_up) / max(1, total_steps - warm_up)
    return lr_mini + 0.5 * (lr_max - lr_mini) * (1 + math.cos(math.pi * progress))
