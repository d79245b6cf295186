from . import state  # noqa: F401
from .engine import (AdamW_FP32OptimParams, AdamW_LowPrecision, initialize_parallel_model,  # noqa: F401
                     initialize_parallel_optimizer, load_checkpoint, neuronx_distributed_config,
                     parallel_config, save_checkpoint)
