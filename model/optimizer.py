"""``model.optimizer`` of the reference: host-offloaded and GPU-sharded AdamW."""
from create_llm_by_cupy_b200.optim.optimizer import ZeRO_Adam_Offload, ZeRO_Adam_ShardedGPU, cosine_lr  # noqa: F401
