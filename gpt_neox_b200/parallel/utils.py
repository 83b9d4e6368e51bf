"""Small helpers of the tensor-parallel layers (megatron/mpu/utils.py:29-96)."""
from __future__ import annotations

import torch


def ensure_divisibility(numerator: int, denominator: int):
    assert numerator % denominator == 0, f"{numerator} is not divisible by {denominator}"


def divide(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False):
    size = divide(tensor.size(-1), num_partitions)
    parts = torch.split(tensor, size, dim=-1)
    return tuple(p.contiguous() for p in parts) if contiguous_split_chunks else parts


def split_tensor_along_any_dim(tensor, num_partitions, seq_dim, contiguous_split_chunks=False):
    size = divide(tensor.size(seq_dim), num_partitions)
    parts = torch.split(tensor, size, dim=seq_dim)
    return tuple(p.contiguous() for p in parts) if contiguous_split_chunks else parts


class VocabUtility:
    """[first, last) vocabulary ids owned by a rank when the vocabulary is split in equal chunks."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition_vocab_size, rank, world_size):
        first = rank * per_partition_vocab_size
        return first, first + per_partition_vocab_size

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size, rank, world_size):
        return VocabUtility.vocab_range_from_per_partition_vocab_size(
            divide(global_vocab_size, world_size), rank, world_size)
