"""Parallel primitives ("mpu"): groups, region mappings, tensor-parallel layers, vocab-parallel
cross-entropy, batch broadcast, RNG streams and activation checkpointing."""
from .cross_entropy import vocab_parallel_cross_entropy  # noqa: F401
from .data import broadcast_data  # noqa: F401
from .layers import (ColumnParallelLinear, ParallelRelativePositionBias, RowParallelLinear,  # noqa: F401
                     VocabParallelEmbedding)
from .mappings import *  # noqa: F401,F403
from .random import checkpoint, get_cuda_rng_tracker, model_parallel_cuda_manual_seed  # noqa: F401
from .state import *  # noqa: F401,F403
from .state import (PipeModelDataParallelTopology, ProcessTopology, destroy_model_parallel,  # noqa: F401
                    initialize_model_parallel, model_parallel_is_initialized)
from .utils import VocabUtility, divide, split_tensor_along_last_dim  # noqa: F401
