"""``Cupa_ver4``: decoder-only transformer (pre-norm RMSNorm, RoPE, GQA, SwiGLU, tied or untied LM
head with chunked cross-entropy) with explicit ``forward`` / ``backward`` that interleave with a
ZeRO manager, plus ``predict``, KV-cache ``generate`` / ``chat_generate`` and weight I/O.

Same surface as the reference model (model/model.py:12-99 ctor, :189 forward, :266 backward,
:418 predict, :439 generate, :483 chat_generate, :539 make_mask, :551 load_weights_from_flat_file,
:574 self_link_params, :591 link_params). What differs is what the reference leaves broken or
fixed in stone: generation/predict work (and decode with a KV cache instead of one full forward
per token), the FFN width, embedding tying, RoPE base, Adam betas, dtype and seed are
configurable, and nothing of size [T, T] is ever allocated.

Parameter order in ``self.params`` (kept from the reference, model/model.py:85-97,31-33):
per block ``[W_KQV, W_O, W_gate_val, W_out, gamma1, gamma2]``, then the embedding table, then the
LM head (only when ``tie_embeddings`` is False), then the final norm gamma.
"""
from __future__ import annotations

import gzip
import pickle

import numpy as np
import torch

from ..ops import functional as F
from .layers import (ChunkedCrossEntropy_Share, GroupedQueryAttention, RMSNorm, SwiGLU, TimeDropout,
                     TimeEmbedding_shard, init_weight)
from .sampling import apply_repetition_penalty, top_p_sampling

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32}


class _LocalManager:
    """Manager protocol for a model whose parameters simply stay resident (one process, no
    sharding): gathers return the live tensors, gradients stay in ``layer.grads``."""

    enable_grad_bucket = False
    enable_param_prefetch = False
    enable_forward_param_prefetch = False
    enable_backward_param_prefetch = False

    def __init__(self, model):
        self.model = model
        self.emb_grad = None
        self.head_grad = None

    def gather_embedding(self):
        return self.model.Af_Em_para[0]

    get_live_embedding = gather_embedding

    def gather_head(self):
        return self.model.head_para[0] if self.model.head_para is not None else self.model.Af_Em_para[0]

    def release_embedding(self):
        pass

    def gather_module(self, m):
        pass

    def gather_modules(self, ms):
        pass

    def release_module(self, m):
        pass

    def release_modules(self, ms):
        pass

    def prefetch_modules(self, ms, tag=None):
        pass

    def wait_modules(self, ms):
        pass

    def begin_grad_bucket(self, tag=None, modules=None):
        pass

    def grad_views(self, module):
        return None

    def add_grads_to_bucket(self, params, grads):
        pass

    def accumulate_grads(self, params, grads):
        pass

    def flush_grad_bucket_async(self, tag=None):
        pass

    def embedding_grad_view(self, which="embedding"):
        W = self.gather_embedding() if which == "embedding" else self.gather_head()
        g = torch.zeros_like(W)
        if which == "embedding":
            self.emb_grad = g
        else:
            self.head_grad = g
        return g

    def flush_embedding_grad_bucket_async(self, tag=None):
        pass

    def progress_async_reduces(self, max_pending=8, force=False):
        pass


class Cupa_ver4:
    def __init__(self, model_dic: dict, param_path: str | None = None, device=None):
        d = model_dic
        self.model_dic = dict(d)
        self.layernum = int(d["layer_num"])
        self.time_size = int(d["time_size"])
        self.hidden_size = int(d["hidden_size"])
        self.dropout_rate = float(d.get("dropout_rate", 0))
        self.padding_id = int(d["padding_id"]) if d.get("padding_id") is not None else -1
        self.vocab_size = int(d["vocab_size"])
        self.kv_head = int(d["kv_head"])
        self.q_head = int(d["q_head"])
        self.half_float = bool(d.get("half_float", True))
        self.ffn_size = d.get("ffn_size")
        self.tie_embeddings = bool(d.get("tie_embeddings", True))
        self.rope_base = float(d.get("rope_base", 10000.0))
        self.init_std = d.get("init_std")
        self.seed = int(d.get("seed", 0))
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        default_dtype = "bf16" if (self.half_float and self.device.type == "cuda") else "fp32"
        self.dtype = _DTYPES[str(d.get("dtype", default_dtype))]
        self.head_dim = self.hidden_size // self.q_head

        # Weights are drawn from one seeded generator in ``params`` order, so every rank (and the
        # NumPy oracle, which reads them back) starts from identical values.
        gen = torch.Generator(device="cpu" if self.device.type == "cpu" or d.get("init_on_cpu") else self.device)
        gen.manual_seed(self.seed)
        self._gen = gen

        chunk = int(d.get("ce_chunk_size", 8192))
        self.AF_Cross_loss = ChunkedCrossEntropy_Share(self.padding_id, chunk, self.dtype,
                                                      cache_logits=bool(d.get("ce_cache_logits", False)))
        self.embed = TimeEmbedding_shard(self.padding_id, self.dtype)
        self.params = []
        self._initialize_layers()
        emb_std = self.init_std if self.init_std is not None else 0.02
        self.Af_Em_para = [init_weight((self.vocab_size, self.hidden_size), emb_std, self.dtype, self.device, gen)]
        self.params += self.Af_Em_para
        self.head_para = None
        if not self.tie_embeddings:
            self.head_para = [init_weight((self.vocab_size, self.hidden_size), emb_std, self.dtype, self.device, gen)]
            self.params += self.head_para
        self.params += self.norm_.params
        self.one_cycle_num = len(self.layers) // self.layernum
        self.grads = []
        self.keep_layer_num = 1
        if param_path is not None:
            self.load_weights_from_flat_file(param_path)
            self.self_link_params()
        self._apply_runtime_options(d)

    # ------------------------------------------------------------------ construction
    def _initialize_layers(self):
        self.layers = []
        kw = dict(dtype=self.dtype, device=self.device, generator=self._gen, init_std=self.init_std)
        if self.dropout_rate != 0:
            self.dropout_ = TimeDropout(self.dropout_rate, self.dtype)
        for _ in range(self.layernum):
            gqa = GroupedQueryAttention(self.hidden_size, self.time_size, self.q_head, self.kv_head, self.layernum,
                                        self.dropout_rate, rope_base=self.rope_base, **kw)
            feed = SwiGLU(self.hidden_size, self.layernum, dropout_rate=self.dropout_rate, ffn_size=self.ffn_size, **kw)
            norm1 = RMSNorm(self.hidden_size, self.dtype, self.device)
            norm2 = RMSNorm(self.hidden_size, self.dtype, self.device)
            for m in (gqa, feed, norm1, norm2):
                self.layers.append(m)
                self.params += m.params
        self.norm_ = RMSNorm(self.hidden_size, self.dtype, self.device)

    def _apply_runtime_options(self, d: dict):
        g = d.get
        self.keep_layer_num = max(1, int(g("keep_layer_num", getattr(self, "keep_layer_num", 1))))
        self.keep_embedding_until_backward = bool(g("keep_embedding_until_backward", True))
        # Keep every block's gathered parameters from the training forward until its backward has used
        # them (one all-gather per unit and step instead of two; the model's bf16 parameters stay
        # resident on every rank during the step - 2.3 GB for the 1.3 B model).
        self.keep_params_until_backward = bool(g("keep_params_until_backward", False))
        # On a 180 GB part keeping activations beats recomputing them; the reference's defaults
        # (False) remain selectable.
        self.gqa_cache_out_value = bool(g("gqa_cache_out_value", True))
        self.gqa_cache_kqv = bool(g("gqa_cache_kqv", True))
        self.gqa_cache_attn = bool(g("gqa_cache_attn", False))
        self.swiglu_cache_gate = bool(g("swiglu_cache_gate", True))
        self.zero3_param_prefetch = bool(g("zero3_param_prefetch", True))
        self.zero3_forward_param_prefetch = bool(g("zero3_forward_param_prefetch", self.zero3_param_prefetch))
        self.zero3_backward_param_prefetch = bool(g("zero3_backward_param_prefetch", self.zero3_param_prefetch))
        self.zero3_reduce_progress = bool(g("zero3_reduce_progress", True))
        self.zero3_max_pending_reduces = int(g("zero3_max_pending_reduces", 8))
        self.zero3_grad_bucket = bool(g("zero3_grad_bucket", True))
        self.zero3_grad_bucket_flatten = bool(g("zero3_grad_bucket_flatten", True))
        self.zero3_grad_bucket_max_bytes = int(g("zero3_grad_bucket_max_bytes", 256 * 1024 * 1024))
        self.zero3_owner_grad_bucket = bool(g("zero3_owner_grad_bucket", True))
        self.zero3_embedding_grad_bucket = bool(g("zero3_embedding_grad_bucket", True))
        self.zero3_embedding_grad_bucket_max_bytes = int(g("zero3_embedding_grad_bucket_max_bytes", 64 * 1024 * 1024))
        self.zero3_sync_gather = bool(g("zero3_sync_gather", False))
        self.zero3_sync_after_each_microbatch = bool(g("zero3_sync_after_each_microbatch", False))
        # multi-GPU data plane of the training worker: peer-memory kernels / copy engines (default) or NCCL
        self.zero3_fused_collectives = bool(g("zero3_fused_collectives", True))
        self.zero3_gather_mode = str(g("zero3_gather_mode", "copy"))
        self.zero3_reduce_mode = str(g("zero3_reduce_mode", "copy"))
        self.zero3_gather_stream = bool(g("zero3_gather_stream", True))
        self.grad_bucket_elems = int(g("grad_bucket_elems", 25_000_000))
        self.zero3_early_bucket_flush = bool(g("zero3_early_bucket_flush", False))
        backend = str(g("flash_backend", "b200"))
        for layer in self.layers:
            if isinstance(layer, GroupedQueryAttention):
                layer.cache_out_value = self.gqa_cache_out_value
                layer.cache_kqv = self.gqa_cache_kqv
                layer.cache_attn = self.gqa_cache_attn
                # "cupy" / "triton" name the reference's flash paths; all of them map onto the
                # native kernels here, "none" keeps the dense verification path.
                layer.flash_backend = "none" if backend == "none" else "b200"
            elif isinstance(layer, SwiGLU):
                layer.cache_gate = self.swiglu_cache_gate

    # ------------------------------------------------------------------ structure helpers
    def block_modules(self, b: int):
        s = b * self.one_cycle_num
        return self.layers[s:s + self.one_cycle_num]

    def _make_layer_groups(self):
        """[(first block, last block + 1, [modules])] with ``keep_layer_num`` blocks per gather."""
        groups = []
        for b0 in range(0, self.layernum, self.keep_layer_num):
            b1 = min(b0 + self.keep_layer_num, self.layernum)
            mods = []
            for b in range(b0, b1):
                mods += self.block_modules(b)
            groups.append((b0, b1, mods))
        return groups

    def unit_defs(self):
        """[(unit name, [param indices])] used by the ZeRO layout: one unit per block, one for the
        embedding table, one for the untied LM head, one for the final norm."""
        defs = []
        per = 6
        for b in range(self.layernum):
            # Inside a block's unit the two norm gains come first, then the attention weights, then the MLP
            # weights: the MLP part (the first gradients a block's backward completes) is then one contiguous
            # tail that can be reduced ahead of the rest, and the rest is one contiguous head.
            i0 = b * per
            defs.append((f"block{b}", [i0 + 4, i0 + 5, i0, i0 + 1, i0 + 2, i0 + 3]))
        i = self.layernum * per
        defs.append(("embedding", [i]))
        i += 1
        if not self.tie_embeddings:
            defs.append(("lm_head", [i]))
            i += 1
        defs.append(("final_norm", [i]))
        return defs

    def unit_modules(self):
        """unit name -> list of (module, param position in module.params, param index)."""
        out = {}
        idx = 0
        for b in range(self.layernum):
            ent = []
            for m in self.block_modules(b):
                for j in range(len(m.params)):
                    ent.append((m, j, idx))
                    idx += 1
            out[f"block{b}"] = ent
        out["embedding"] = [(self, "Af_Em_para", idx)]
        idx += 1
        if not self.tie_embeddings:
            out["lm_head"] = [(self, "head_para", idx)]
            idx += 1
        out["final_norm"] = [(self.norm_, 0, idx)]
        return out

    def param_count(self) -> int:
        return sum(int(np.prod(p.shape)) for p in self.params if p is not None)

    # ------------------------------------------------------------------ masks
    def make_mask(self, padding_box: torch.Tensor) -> torch.Tensor:
        """Additive [B, 1, 1, T] key mask: -inf where position >= valid length
        (model/model.py:539-548). The flash kernels take the lengths directly; this dense form is
        for the verification path and for callers of the reference API."""
        T = self.time_size
        pos = torch.arange(T, device=padding_box.device)[None, :]
        bad = pos >= padding_box[:, None]
        m = torch.zeros(bad.shape, dtype=torch.float32, device=padding_box.device)
        m.masked_fill_(bad, float("-inf"))
        return m[:, None, None, :]

    # ------------------------------------------------------------------ training forward / backward
    def _use_forward_prefetch(self, manager) -> bool:
        return bool(getattr(manager, "enable_forward_param_prefetch", False)) and self.zero3_forward_param_prefetch

    def _use_backward_prefetch(self, manager) -> bool:
        return bool(getattr(manager, "enable_backward_param_prefetch", False)) and self.zero3_backward_param_prefetch

    def forward(self, x, t, x_pa=None, manager=None, train_flg: bool = True):
        """x, t: int token ids [B, T]; x_pa: int32 [B] valid key length per sequence (keys at
        positions >= x_pa are masked) or None. Returns the mean CE loss as a device scalar."""
        manager = manager if manager is not None else self._local_manager()
        self._manager = manager
        manager.phase = "fwd"
        self.grads = []
        B, T = x.shape
        self._BT = (B, T)
        valid_len = None if x_pa is None else x_pa.to(torch.int32)

        W = manager.gather_embedding()
        h = self.embed.forward(W, x, train_flg)
        if self.dropout_rate != 0:
            h = self.dropout_.forward(h, train_flg)

        groups = self._make_layer_groups()
        use_prefetch = self._use_forward_prefetch(manager)
        if use_prefetch and groups:
            manager.prefetch_modules(groups[0][2], tag="fwd_group_0")
        for gi, (_, _, mods) in enumerate(groups):
            if use_prefetch:
                manager.wait_modules(mods)
                if gi + 1 < len(groups):
                    manager.prefetch_modules(groups[gi + 1][2], tag=f"fwd_group_{gi + 1}")
            else:
                manager.gather_modules(mods)
            for s in range(0, len(mods), self.one_cycle_num):
                gqa, feed, norm1, norm2 = mods[s:s + self.one_cycle_num]
                h = gqa.forward(norm1.forward(h, train_flg), B, T, valid_len, residual=h, train_flg=train_flg)
                h = feed.forward(norm2.forward(h, train_flg), residual=h, train_flg=train_flg)
            if not (train_flg and self.keep_params_until_backward):
                manager.release_modules(mods)
        self.x_pa = x_pa

        manager.gather_module(self.norm_)
        h = self.norm_.forward(h, train_flg)
        manager.release_module(self.norm_)

        Wh = manager.gather_head()
        loss = self.AF_Cross_loss.forward(h, t, Wh, train_flg)
        if not train_flg or not self.keep_embedding_until_backward:
            manager.release_embedding()
        return loss

    def backward(self, GradScale: float = 1.0, manager=None):
        manager = manager if manager is not None else getattr(self, "_manager", None) or self._local_manager()
        manager.phase = "bwd"
        W = manager.get_live_embedding()
        if W is None:
            W = manager.gather_embedding()
        Wh = manager.gather_head()

        groups = self._make_layer_groups()
        use_prefetch = self._use_backward_prefetch(manager)
        if use_prefetch and groups:
            # issued before the (heavy) CE backward so the gather hides under it
            manager.prefetch_modules(groups[-1][2], tag=f"bwd_group_{len(groups) - 1}")

        which_head = "embedding" if self.tie_embeddings else "lm_head"
        head_grad = manager.embedding_grad_view(which_head)
        dx = self.AF_Cross_loss.backward(Wh, GradScale, grad_writer=lambda s, e: head_grad[s:e])
        self._maybe_progress_reduces(manager)
        if not self.tie_embeddings:
            manager.flush_embedding_grad_bucket_async(tag="lm_head")
            emb_grad = manager.embedding_grad_view("embedding")
            emb_grad.zero_()
        else:
            emb_grad = head_grad

        manager.gather_module(self.norm_)
        manager.begin_grad_bucket(tag="final_norm", modules=[self.norm_])
        dx = self.norm_.backward(dx, grad_out=manager.grad_views(self.norm_))
        manager.add_grads_to_bucket(self.norm_.params, self.norm_.grads)
        manager.flush_grad_bucket_async(tag="final_norm")
        manager.release_module(self.norm_)
        local_grads = {id(self.norm_): self.norm_.grads}

        for gi in range(len(groups) - 1, -1, -1):
            mods = groups[gi][2]
            if use_prefetch:
                manager.wait_modules(mods)
                if gi > 0:
                    manager.prefetch_modules(groups[gi - 1][2], tag=f"bwd_group_{gi - 1}")
            else:
                manager.gather_modules(mods)
            for s in range(len(mods) - self.one_cycle_num, -1, -self.one_cycle_num):
                gqa, feed, norm1, norm2 = mods[s:s + self.one_cycle_num]
                manager.begin_grad_bucket(tag=f"block_{gi}_{s}", modules=[gqa, feed, norm1, norm2])
                dn2 = feed.backward(dx, grad_out=manager.grad_views(feed))
                if hasattr(manager, "flush_grad_ranges_async"):
                    # the MLP weight gradients are complete once the side stream has run them: their part of
                    # the bucket is reduced while the attention half of the block is still in backward
                    manager.flush_grad_ranges_async([feed], tag=f"block_{gi}_{s}_mlp")
                dx = norm2.backward(dn2, add=dx, grad_out=manager.grad_views(norm2))
                dn1 = gqa.backward(dx, grad_out=manager.grad_views(gqa))
                dx = norm1.backward(dn1, add=dx, grad_out=manager.grad_views(norm1))
                F.wgrad_join(dx.device)      # weight-gradient GEMMs of this block (side stream) are in the bucket
                for m in (feed, norm2, gqa, norm1):
                    manager.add_grads_to_bucket(m.params, m.grads)
                    local_grads[id(m)] = m.grads
                manager.flush_grad_bucket_async(tag=f"block_{gi}_{s}")
                self._maybe_progress_reduces(manager)
            manager.release_modules(mods)

        if self.dropout_rate != 0:
            dx = self.dropout_.backward(dx)
        self.embed.backward(emb_grad, dx)
        manager.flush_embedding_grad_bucket_async(tag="embedding")
        manager.release_embedding()

        if isinstance(manager, _LocalManager):
            self.grads = []
            for m in self.layers:
                self.grads += local_grads[id(m)]
            self.grads.append(manager.emb_grad)
            if not self.tie_embeddings:
                self.grads.append(manager.head_grad)
            self.grads += local_grads[id(self.norm_)]
        return None

    def _maybe_progress_reduces(self, manager):
        if self.zero3_reduce_progress and hasattr(manager, "progress_async_reduces"):
            manager.progress_async_reduces(max_pending=self.zero3_max_pending_reduces)

    def _local_manager(self):
        m = getattr(self, "_local_mgr", None)
        if m is None:
            m = self._local_mgr = _LocalManager(self)
        return m

    # ------------------------------------------------------------------ inference
    def predict(self, x, t, x_pa=None, manager=None):
        """Loss of a batch without keeping anything for backward (validation)."""
        return self.forward(x, t, x_pa, manager, train_flg=False)

    def logits(self, x, manager=None) -> torch.Tensor:
        """Full-sequence fp32 logits [B, T, V] (no cache); for tests and scoring."""
        manager = manager if manager is not None else self._local_manager()
        B, T = x.shape
        W = manager.gather_embedding()
        h = self.embed.forward(W, x, False)
        for b in range(self.layernum):
            gqa, feed, norm1, norm2 = self.block_modules(b)
            manager.gather_modules([gqa, feed, norm1, norm2])
            h = gqa.forward(norm1.forward(h, False), B, T, None, residual=h, train_flg=False)
            h = feed.forward(norm2.forward(h, False), residual=h, train_flg=False)
            manager.release_modules([gqa, feed, norm1, norm2])
        manager.gather_module(self.norm_)
        h = self.norm_.forward(h, False)
        manager.release_module(self.norm_)
        out = F.gemm(h, manager.gather_head(), trans_b=True, out_dtype=torch.float32)
        return out.view(B, T, self.vocab_size)

    @torch.no_grad()
    def generate(self, prompt, start_id=None, end_id=None, padding_id=None, temp: float = 0.7, top: float = 0.9,
                 penalty: float = 1.2, max_new_tokens: int | None = None, greedy: bool = False, seed: int | None = None):
        """Autoregressive decoding with a KV cache (reference intent: model/model.py:439-480).

        ``prompt``: list of token ids. The sequence is ``[start_id] + prompt`` when ``start_id`` is
        given. One prefill pass fills the cache; every further token costs one single-position
        pass through the decode-attention kernel. Sampling: pad id excluded, repetition penalty,
        temperature, nucleus (top-p) with a probability-weighted draw; ``greedy`` takes the argmax.
        Stops at ``end_id`` or when the context (``time_size``) is full. Parameters must be
        resident (single process), as in the reference.
        """
        pad = self.padding_id if padding_id is None else padding_id
        toks = ([int(start_id)] if start_id is not None else []) + [int(p) for p in prompt]
        if not toks:
            raise ValueError("generate needs at least one token of context")
        Tmax = self.time_size
        toks = toks[:Tmax - 1]
        budget = Tmax - len(toks) if max_new_tokens is None else min(max_new_tokens, Tmax - len(toks))
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.device)
            gen.manual_seed(seed)
        dev, dt = self.device, self.dtype
        kc = [torch.zeros((1, self.kv_head, Tmax, self.head_dim), dtype=dt, device=dev) for _ in range(self.layernum)]
        vc = [torch.zeros_like(kc[0]) for _ in range(self.layernum)]
        W = self.Af_Em_para[0]
        Wh = self.head_para[0] if self.head_para is not None else W

        T0 = len(toks)
        ids = torch.tensor(toks, dtype=torch.int32, device=dev)
        h = F.embedding_fwd(W, ids, -1)
        for b in range(self.layernum):
            gqa, feed, norm1, norm2 = self.block_modules(b)
            h = gqa.prefill(norm1.forward(h, False), 1, T0, kc[b], vc[b], residual=h)
            h = feed.forward(norm2.forward(h, False), residual=h, train_flg=False)
        h_last = self.norm_.forward(h[T0 - 1:T0], False)
        out = []
        lens = torch.zeros(1, dtype=torch.int32, device=dev)
        for _ in range(budget):
            logits = F.gemm(h_last, Wh, trans_b=True, out_dtype=torch.float32)[0]
            if 0 <= pad < self.vocab_size:
                logits[pad] = float("-inf")
            if greedy:
                nxt = int(torch.argmax(logits))
            else:
                logits = apply_repetition_penalty(logits, toks + out, penalty)
                nxt = top_p_sampling(logits, temp, top, generator=gen)
            out.append(nxt)
            pos = T0 + len(out) - 1
            if (end_id is not None and nxt == end_id) or pos >= Tmax - 1:
                break
            tok = torch.tensor([nxt], dtype=torch.int32, device=dev)
            h = F.embedding_fwd(W, tok, -1)
            lens.fill_(pos + 1)
            for b in range(self.layernum):
                gqa, feed, norm1, norm2 = self.block_modules(b)
                h = gqa.decode_step(norm1.forward(h, False), pos, kc[b], vc[b], lens, residual=h)
                h = feed.forward(norm2.forward(h, False), residual=h, train_flg=False)
            h_last = self.norm_.forward(h, False)
        return out

    def chat_generate(self, prompt, user_id, bot_id, end_id, padding_id=None, **kw):
        """Wraps the prompt as ``[user_id] + prompt + [end_id] + [bot_id]`` (model/model.py:483-536)."""
        return self.generate([user_id] + list(prompt) + [end_id, bot_id], None, end_id, padding_id, **kw)

    def add_words(self, n_new: int):
        """Grow the vocabulary by ``n_new`` rows drawn N(0, 0.02) (embedding and untied head)."""
        extra = init_weight((n_new, self.hidden_size), 0.02, self.dtype, self.device, self._gen)
        self.Af_Em_para[0] = torch.cat([self.Af_Em_para[0], extra], 0)
        if self.head_para is not None:
            extra2 = init_weight((n_new, self.hidden_size), 0.02, self.dtype, self.device, self._gen)
            self.head_para[0] = torch.cat([self.head_para[0], extra2], 0)
        self.vocab_size += n_new
        self._rebuild_params()

    # ------------------------------------------------------------------ weights I/O
    def _rebuild_params(self):
        self.params = []
        for m in self.layers:
            self.params += m.params
        self.params += self.Af_Em_para
        if self.head_para is not None:
            self.params += self.head_para
        self.params += self.norm_.params

    def link_params(self, new_params):
        """Re-bind every layer's ``params`` to the tensors in ``new_params`` (``params`` order).
        ``None`` entries detach a parameter (what a ZeRO manager does between gathers)."""
        assert len(new_params) == len(self.params)
        i = 0
        for m in self.layers:
            for j in range(len(m.params)):
                m.params[j] = new_params[i]
                i += 1
        self.Af_Em_para[0] = new_params[i]
        i += 1
        if self.head_para is not None:
            self.head_para[0] = new_params[i]
            i += 1
        self.norm_.params[0] = new_params[i]
        self.params = list(new_params)

    def self_link_params(self):
        self.link_params(list(self.params))

    def flat_params(self) -> torch.Tensor:
        """All parameters concatenated in ``params`` order (the flat checkpoint format)."""
        return torch.cat([p.reshape(-1) for p in self.params])

    def load_flat(self, flat: torch.Tensor):
        off = 0
        new = []
        for p in self.params:
            n = p.numel()
            new.append(flat[off:off + n].view(p.shape).to(device=self.device, dtype=self.dtype).clone())
            off += n
        if off != flat.numel():
            raise ValueError(f"flat parameter file has {flat.numel()} elements, model needs {off}")
        self.link_params(new)

    def load_weights_from_flat_file(self, path: str):
        """Load a gzip-pickled flat array of all parameters in ``params`` order — the one resume
        format the reference can read (model/model.py:551-571)."""
        with gzip.open(path, "rb") as f:
            obj = pickle.load(f)
        if isinstance(obj, dict):
            obj = obj.get("flat_params_f16", obj.get("flat_params"))
        arr = np.asarray(obj)
        if arr.dtype == np.uint16:          # bf16 stored as raw bits
            flat = torch.from_numpy(arr.astype(np.int16)).view(torch.bfloat16)
        else:
            flat = torch.from_numpy(arr.astype(np.float32))
        self.load_flat(flat)

    def save_weights_to_flat_file(self, path: str):
        flat = self.flat_params().detach().float().cpu().numpy().astype(np.float16)
        with gzip.open(path, "wb") as f:
            pickle.dump(flat, f, protocol=pickle.HIGHEST_PROTOCOL)


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0, device="cpu"):
    """cos/sin tables [end, dim/2] (model/model.py:640-645), fp32."""
    return F.rope_table(end, dim, theta, device)
