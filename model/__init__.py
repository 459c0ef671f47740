"""Reference-compatible import surface: ``from model.ZeRO3 import TrainMultiGPU`` and friends
resolve to the B200-native implementations in ``create_llm_by_cupy_b200``."""
