"""Vocab-parallel softmax cross-entropy.

Same result as megatron/mpu/cross_entropy.py:27-112 (per-token loss over a vocabulary sharded
across the tensor-parallel group), with one packed cross-rank combine of three floats per token
instead of three all-reduces, no fp32 copy of the logits, and the gradient written over the
logits buffer in backward.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .gemm import LAUNCHES


def _combine_stats(stats: torch.Tensor, group) -> tuple[torch.Tensor, torch.Tensor]:
    """stats [rows, 3] = (local max, local sum-exp rel. to that max, local target logit).
    Returns (lse, target) after combining across ``group``."""
    if group is not None and dist.get_world_size(group) > 1:
        ws = dist.get_world_size(group)
        # one packed exchange of (max, sum-exp, target logit) per row instead of three all-reduces
        # (megatron/mpu/cross_entropy.py:33,68,78); over peer memory when the group has a symmetric workspace
        from ..comm.collectives import all_gather_dim
        flat = all_gather_dim(stats.contiguous(), 0, group=group)
        gathered = flat.view((ws,) + tuple(stats.shape))
        m = gathered[..., 0]
        gm = m.max(dim=0).values
        s = (gathered[..., 1] * torch.exp(m - gm)).sum(0)
        t = gathered[..., 2].sum(0)
    else:
        gm, s, t = stats[:, 0], stats[:, 1], stats[:, 2]
    return gm + torch.log(s), t


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        assert l2.stride(1) == 1
        lab = labels.reshape(-1).contiguous()
        rows = l2.shape[0]
        stats = torch.empty((rows, 3), device=logits.device, dtype=torch.float32)
        dtype = 1 if logits.dtype == torch.float32 else 0
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(l2).nx_ce_fwd(_lib.ptr(l2), _lib.ptr(lab), _lib.ptr(stats), rows, V, l2.stride(0),
                                        int(vocab_start), dtype, _lib.stream()), "nx_ce_fwd")
        lse, tgt = _combine_stats(stats, group)
        ctx.save_for_backward(l2, lab, lse)
        ctx.vocab_start, ctx.dtype, ctx.shape = int(vocab_start), dtype, logits.shape
        return (lse - tgt).view(labels.shape)

    @staticmethod
    def backward(ctx, gloss):
        l2, lab, lse = ctx.saved_tensors
        rows, V = l2.shape
        g = gloss.reshape(-1).float().contiguous()
        # The gradient overwrites the logits buffer when it is 16-bit (it is dead after this op).
        out = l2 if ctx.dtype == 0 else torch.empty(l2.shape, device=l2.device, dtype=torch.bfloat16)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(l2).nx_ce_bwd(_lib.ptr(l2), _lib.ptr(lab), _lib.ptr(lse), _lib.ptr(g), _lib.ptr(out),
                                        rows, V, l2.stride(0), out.stride(0), ctx.vocab_start, ctx.dtype,
                                        _lib.stream()), "nx_ce_bwd")
        if ctx.dtype != 0:
            out = out.float()
        return out.view(ctx.shape), None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int = 0,
                                 group=None) -> torch.Tensor:
    """Per-token loss; ``logits`` [..., V_local] holds vocabulary ids
    [vocab_start, vocab_start + V_local) of the full vocabulary."""
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float16, torch.float32):
        if labels.device != logits.device or labels.dtype != torch.int64:
            raise _lib.KernelError(f"cross_entropy: labels must be int64 on {logits.device}, got {labels.dtype} "
                                   f"on {labels.device}")
        return _VocabParallelCE.apply(logits, labels, vocab_start, group)
    if logits.is_cuda:
        raise _lib.KernelError(f"cross_entropy: unsupported CUDA dtype {logits.dtype}")
    return _ref_vocab_parallel_ce(logits, labels, vocab_start, group)


class _RefCE(torch.autograd.Function):
    """PyTorch statement of the same algorithm (CPU / gloo runs and the oracle)."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group):
        lf = logits.float()
        V = lf.shape[-1]
        m = lf.max(dim=-1).values
        s = torch.exp(lf - m.unsqueeze(-1)).sum(-1)
        local = labels - vocab_start
        inside = (local >= 0) & (local < V)
        idx = local.clamp(0, V - 1)
        t = torch.where(inside, lf.gather(-1, idx.unsqueeze(-1)).squeeze(-1), torch.zeros_like(m))
        stats = torch.stack([m, s, t], dim=-1).reshape(-1, 3)
        lse, tgt = _combine_stats(stats, group)
        lse = lse.view(labels.shape)
        ctx.save_for_backward(lf, lse, idx, inside)
        ctx.in_dtype = logits.dtype
        return lse - tgt.view(labels.shape)

    @staticmethod
    def backward(ctx, gloss):
        lf, lse, idx, inside = ctx.saved_tensors
        p = torch.exp(lf - lse.unsqueeze(-1))
        onehot = torch.zeros_like(p)
        onehot.scatter_(-1, idx.unsqueeze(-1), inside.unsqueeze(-1).to(p.dtype))
        return ((p - onehot) * gloss.unsqueeze(-1)).to(ctx.in_dtype), None, None, None


def _ref_vocab_parallel_ce(logits, labels, vocab_start=0, group=None):
    return _RefCE.apply(logits, labels, vocab_start, group)
