"""``model.ZeRO2_5`` of the reference: the same launcher / worker with the ZeRO-2.5 manager (a
configurable fraction of the parameters replicated, the rest handled as in ZeRO-3)."""
from create_llm_by_cupy_b200.parallel.trainer import TrainMultiGPU_ZeRO25 as TrainMultiGPU  # noqa: F401
from create_llm_by_cupy_b200.parallel.trainer import Trainer, WorkerFailure, training_worker_nccl_stream  # noqa: F401
from create_llm_by_cupy_b200.parallel.zero import MemoryZeRO2_5Manager  # noqa: F401
from create_llm_by_cupy_b200.utils.checkpoint import save_pickle_gzip_to_drive  # noqa: F401
from create_llm_by_cupy_b200.utils.data import (data_shuffle, get_batch, load_input_ids_from_drive,  # noqa: F401
                                                 padding_proceccing)
