"""``model.functions`` of the reference: loss-scale controller, initialisers, clipping, memory report."""
from create_llm_by_cupy_b200.utils.functions import (ScaleGrad, ZeRO_clip_grads, clip_coefficient, init_weight,  # noqa: F401
                                                      place_enco, print_memory_status, sigmoid, softmax,
                                                      total_clip_grads, xavier_initialization)
