"""Vocab-parallel cross-entropy over the tensor-parallel group (megatron/mpu/cross_entropy.py:115)."""
from __future__ import annotations

from ..ops.cross_entropy import vocab_parallel_cross_entropy as _vpce
from . import state as mpu
from .utils import VocabUtility


def vocab_parallel_cross_entropy(vocab_parallel_logits, target):
    """Per-token loss; ``vocab_parallel_logits`` [..., V / tp] is this rank's vocabulary shard."""
    ws, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
    v_local = vocab_parallel_logits.shape[-1]
    start, _ = VocabUtility.vocab_range_from_per_partition_vocab_size(v_local, rank, ws)
    group = mpu.get_model_parallel_group() if ws > 1 else None
    return _vpce(vocab_parallel_logits, target, start, group)
