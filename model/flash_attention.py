"""``model.flash_attention`` of the reference. The CuPy-tiled and Triton entry points map onto the
native causal GQA kernels (``[B, T, heads, D]`` layout, RoPE optionally fused)."""
from create_llm_by_cupy_b200.ops.functional import decode_attn, flash_attn_bwd, flash_attn_fwd  # noqa: F401

cupy_flash_gqa_forward = flash_attn_fwd
cupy_flash_gqa_backward = flash_attn_bwd
triton_flash_gqa_forward = flash_attn_fwd
