"""``model.fast_layers`` of the reference: layers with hand-written forward / backward, and the two rotary
helpers with the reference's signatures (model/fast_layers.py:27-70)."""
import torch

from create_llm_by_cupy_b200.models.layers import (ChunkedCrossEntropy_Share, GroupedQueryAttention, RMSNorm,  # noqa: F401
                                                    SoftMax, SwiGLU, TimeDropout, TimeEmbedding_shard, init_weight)
from create_llm_by_cupy_b200.ops import functional as _F


def precompute_freqs_cis(dim, end, theta=10000.0, dtype=torch.float32, device="cpu"):
    """cos / sin tables ``[end, dim / 2]`` with ``freq_j = theta^(-2j / dim)``, computed in fp32."""
    cos, sin = _F.rope_table(int(end), int(dim), float(theta), device)
    return cos.to(dtype), sin.to(dtype)


def apply_rotary_pos_emb_inplace(x, cos, sin):
    """Half-split rotary embedding of ``x [..., T, D]`` (e.g. ``[B, heads, T, D]``) in place, position =
    index along the second-to-last axis; ``cos`` / ``sin`` are ``[T, D / 2]`` (or broadcastable to
    ``[..., T, D / 2]``). Passing ``-sin`` undoes the rotation, which is how the reference's backward uses it."""
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos.to(torch.float32), sin.to(torch.float32)
    a, b = x1.float(), x2.float()
    n1, n2 = a * c - b * s, b * c + a * s            # both halves from the old values before either is written
    x1.copy_(n1.to(x.dtype))
    x2.copy_(n2.to(x.dtype))
    return x
