"""``model.model`` of the reference: the transformer and its sampling helpers."""
from create_llm_by_cupy_b200.models.model import Cupa_ver4, precompute_freqs_cis  # noqa: F401
from create_llm_by_cupy_b200.models.sampling import (apply_repetition_penalty, softmax_with_temperature,  # noqa: F401
                                                      top_p_sampling)
