"""``model.fast_layers`` of the reference: layers with hand-written forward / backward."""
from create_llm_by_cupy_b200.models.layers import (ChunkedCrossEntropy_Share, GroupedQueryAttention, RMSNorm,  # noqa: F401
                                                    SoftMax, SwiGLU, TimeDropout, TimeEmbedding_shard)
from create_llm_by_cupy_b200.ops.functional import rope_inplace as apply_rotary_pos_emb_inplace  # noqa: F401
from create_llm_by_cupy_b200.ops.functional import rope_table as precompute_freqs_cis  # noqa: F401
