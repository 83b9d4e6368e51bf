"""Elastic batch configuration: one global batch size that stays valid over a range of GPU counts.

The reference passes its ``elasticity`` block through to DeepSpeed (megatron/neox_arguments/deepspeed_args.py:229).
Here the block is acted on when the batch keys are derived: with ``elasticity.enabled`` the train batch size is
chosen once from ``max_train_batch_size`` and the allowed ``micro_batch_sizes`` so that as many data-parallel
sizes as possible between ``min_gpus`` and ``max_gpus`` divide it, and a restart on another number of GPUs
(ZeRO shards are re-partitioned at load) keeps the SAME global batch, with only the micro-batch size and
the accumulation steps changing.

Block keys: ``enabled``, ``max_train_batch_size``, ``micro_batch_sizes``, ``min_gpus`` (1), ``max_gpus`` (10000),
``prefer_larger_batch`` (true), ``num_gpus_per_node`` (1: valid GPU counts are multiples of it),
``model_parallel_size`` (1), ``ignore_non_elastic_batch_info`` (false), ``version``.
"""
from __future__ import annotations

from typing import Dict, List, Tuple


class ElasticityError(ValueError):
    pass


def _divisors(n: int) -> List[int]:
    out, i = set(), 1
    while i * i <= n:
        if n % i == 0:
            out.update((i, n // i))
        i += 1
    return sorted(out)


def valid_gpu_counts(batch: int, micro_batches: List[int], min_gpus: int, max_gpus: int, per_node: int = 1) -> List[int]:
    """Data-parallel sizes g for which some allowed micro-batch m gives ``batch == m * g * steps``."""
    ok = set()
    for m in micro_batches:
        if batch % m == 0:
            for g in _divisors(batch // m):
                if min_gpus <= g <= max_gpus and g % per_node == 0:
                    ok.add(g)
    return sorted(ok)


def candidate_batch_sizes(micro_batches: List[int], max_batch: int) -> List[int]:
    """Batch sizes worth scoring: every allowed micro-batch times a number with many divisors (the products
    2^a 3^b 5^c 7^d with non-increasing exponents), kept within ``max_batch``."""
    rich = set()
    for a in range(0, 14):
        for b in range(0, a + 1):
            for c in range(0, b + 1):
                for d in range(0, c + 1):
                    v = (2 ** a) * (3 ** b) * (5 ** c) * (7 ** d)
                    if v <= max_batch:
                        rich.add(v)
    out = set()
    for m in micro_batches:
        for v in rich:
            if m * v <= max_batch:
                out.add(m * v)
    return sorted(out)


def compute_elastic_config(block: Dict, world_size: int = 0) -> Tuple[int, List[int], int]:
    """-> (train batch size, valid data-parallel sizes, micro-batch size for ``world_size`` or 0).

    ``world_size`` counts data-parallel ranks times ``model_parallel_size`` of the block; with 0 only the
    batch size and the valid sizes are computed."""
    if not block or not block.get("enabled"):
        raise ElasticityError("elasticity is not enabled")
    try:
        max_batch = int(block["max_train_batch_size"])
        micro = sorted({int(m) for m in block["micro_batch_sizes"]})
    except KeyError as e:
        raise ElasticityError(f"elasticity needs the key {e}") from None
    if not micro or any(m <= 0 for m in micro) or max_batch < min(micro):
        raise ElasticityError("elasticity: micro_batch_sizes must be positive and fit in max_train_batch_size")
    min_g, max_g = int(block.get("min_gpus", 1)), int(block.get("max_gpus", 10000))
    if min_g < 1 or max_g < min_g:
        raise ElasticityError("elasticity: need 1 <= min_gpus <= max_gpus")
    per_node = int(block.get("num_gpus_per_node", 1))
    mp = int(block.get("model_parallel_size", 1))
    prefer_larger = bool(block.get("prefer_larger_batch", True))
    best, best_valid = None, []
    for b in candidate_batch_sizes(micro, max_batch):
        valid = valid_gpu_counts(b, micro, min_g, max_g, per_node)
        better = len(valid) > len(best_valid) or (len(valid) == len(best_valid) and best is not None
                                                  and (b > best) == prefer_larger and b != best)
        if best is None or better:
            best, best_valid = b, valid
    if not best_valid:
        raise ElasticityError("elasticity: no batch size fits the given micro-batch sizes and GPU range")
    chosen = 0
    if world_size > 0:
        if world_size % mp:
            raise ElasticityError(f"elasticity: world size {world_size} is not a multiple of model_parallel_size {mp}")
        dp = world_size // mp
        if dp not in best_valid:
            raise ElasticityError(f"elasticity: {dp} data-parallel ranks cannot form batch {best}; valid: {best_valid}")
        fits = [m for m in micro if best % (m * dp) == 0]
        chosen = max(fits) if prefer_larger else min(fits)
    return best, best_valid, chosen
