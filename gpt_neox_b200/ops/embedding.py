"""Vocab-parallel embedding lookup (megatron/mpu/layers.py:186-212): ids outside this rank's
vocabulary range give zero rows; the caller reduces across the tensor-parallel group."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import LAUNCHES


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, vocab_start):
        flat = ids.reshape(-1).contiguous()
        V, H = table.shape
        out = torch.empty((flat.numel(), H), device=table.device, dtype=table.dtype)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(table).nx_embedding_fwd(_lib.ptr(flat), _lib.ptr(table), _lib.ptr(out), flat.numel(), H,
                                               int(vocab_start), V, _lib.stream()), "nx_embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.table, ctx.vocab_start = table, int(vocab_start)
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, gy):
        (flat,) = ctx.saved_tensors
        table = ctx.table
        V, H = table.shape
        g2 = gy.reshape(-1, H).contiguous()
        mg = getattr(table, "main_grad", None)
        target = mg if mg is not None else torch.zeros((V, H), device=table.device, dtype=torch.float32)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(g2).nx_embedding_bwd(_lib.ptr(flat), _lib.ptr(g2), _lib.ptr(target), flat.numel(), H,
                                               ctx.vocab_start, V, _lib.stream()), "nx_embedding_bwd")
        return None, (None if mg is not None else target.to(table.dtype)), None


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    if table.is_cuda and table.dtype in _lib.H16 and table.shape[1] % 8 == 0:
        if ids.device != table.device or ids.dtype != torch.int64:
            raise _lib.KernelError(f"embedding: ids must be int64 on {table.device}, got {ids.dtype} on {ids.device}")
        return _EmbeddingFn.apply(ids, table, vocab_start)
    if table.is_cuda:
        raise _lib.KernelError("embedding: CUDA path needs a bf16 table with H % 8 == 0")
    V = table.shape[0]
    local = ids - vocab_start
    inside = (local >= 0) & (local < V)
    out = F.embedding(local.clamp(0, V - 1), table)
    return out * inside.unsqueeze(-1).to(out.dtype)
