"""``model.ZeRO3`` of the reference: launcher, worker loop, data helpers, checkpoint writer and the
ZeRO-3 manager."""
from create_llm_by_cupy_b200.parallel.trainer import (TrainMultiGPU, Trainer, WorkerFailure,  # noqa: F401
                                                       training_worker_nccl_stream)
from create_llm_by_cupy_b200.parallel.zero import MemoryZeRO3Manager  # noqa: F401
from create_llm_by_cupy_b200.utils.checkpoint import save_pickle_gzip_to_drive  # noqa: F401
from create_llm_by_cupy_b200.utils.data import (data_shuffle, get_batch, load_input_ids_from_drive,  # noqa: F401
                                                 padding_proceccing)
