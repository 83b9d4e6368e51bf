"""Tensor / sequence / expert parallel region mappings: each is a (forward op, backward op) pair.

  copy_to_model_parallel_region          identity        <-> all-reduce
  reduce_from_model_parallel_region      all-reduce      <-> identity
  scatter_to_model_parallel_region       split last dim  <-> all-gather last dim
  gather_from_model_parallel_region      all-gather last <-> split last dim
  reduce_scatter_to_sequence_parallel_region   reduce-scatter(seq) <-> all-gather(seq)
  gather_from_sequence_parallel_region         all-gather(seq)     <-> reduce-scatter(seq)
  scatter_to_sequence_parallel_region          split(seq)          <-> all-gather(seq)
  copy_to_expert_model_parallel_region         slice this rank's experts' rows <-> variable all-gather
  gather_from_expert_model_parallel_region     variable all-gather <-> slice

Same algebra as megatron/mpu/mappings.py:283-499.  The collectives go through ``comm.collectives``,
which issues torch.distributed calls in ``nccl_baseline`` mode (and on CPU/gloo) and the in-kernel
NVLink paths in ``fused`` mode.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state as mpu


def _group():
    return mpu.get_model_parallel_group()


def _ws():
    return mpu.get_model_parallel_world_size()


def _maybe_fp32(x):
    if mpu.get_fp32_allreduce() and x.dtype != torch.float32:
        return x.float(), x.dtype
    return x, None


def _reduce(x):
    if _ws() == 1:
        return x
    y, dt = _maybe_fp32(x)
    from ..comm.collectives import all_reduce
    y = all_reduce(y.contiguous(), group=_group())
    return y.to(dt) if dt is not None else y


def _split(x):
    ws = _ws()
    if ws == 1:
        return x
    size = x.shape[-1] // ws
    return x.split(size, dim=-1)[mpu.get_model_parallel_rank()].contiguous()


def _gather(x):
    ws = _ws()
    if ws == 1:
        return x
    from ..comm.collectives import all_gather_list
    parts = all_gather_list(x.contiguous(), group=_group())
    return torch.cat(parts, dim=-1).contiguous()


def _reduce_scatter_along_seq_dim(x, seq_dim):
    ws = _ws()
    if ws == 1:
        return x
    y, dt = _maybe_fp32(x)
    assert y.shape[seq_dim] % ws == 0
    from ..comm.collectives import reduce_scatter_dim
    out = reduce_scatter_dim(y, seq_dim, group=_group())
    return out.to(dt) if dt is not None else out


def _gather_along_seq_dim(x, seq_dim):
    ws = _ws()
    if ws == 1:
        return x
    from ..comm.collectives import all_gather_dim
    return all_gather_dim(x, seq_dim, group=_group())


def _split_along_seq_dim(x, seq_dim):
    ws = _ws()
    if ws == 1:
        return x
    n = x.shape[seq_dim] // ws
    r = mpu.get_model_parallel_rank()
    return x.narrow(seq_dim, r * n, n).contiguous()


def _dmoe_slice(x, tokens_per_expert):
    if _ws() == 1:
        return x
    return mpu.get_expert_tokens_for_rank(x, tokens_per_expert)


def _dmoe_gather(x, tokens_per_expert):
    """Variable-size all-gather along dim 0: rank r contributes the rows of its experts."""
    ws = _ws()
    if ws == 1:
        return x
    per = tokens_per_expert.numel() // ws
    counts = tokens_per_expert.view(ws, per).sum(-1).tolist()
    parts = [torch.empty((int(c),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device) for c in counts]
    dist.all_gather(parts, x.contiguous(), group=_group())
    return torch.cat(parts, dim=0)


class _CopyToMP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _reduce(g)


class _ReduceFromMP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _reduce(x)

    @staticmethod
    def backward(ctx, g):
        return g


class _ScatterToMP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _split(x)

    @staticmethod
    def backward(ctx, g):
        return _gather(g)


class _GatherFromMP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _gather(x)

    @staticmethod
    def backward(ctx, g):
        return _split(g)


class _ReduceScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        ctx.seq_dim = seq_dim
        return _reduce_scatter_along_seq_dim(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _gather_along_seq_dim(g, ctx.seq_dim), None


class _GatherFromSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        ctx.seq_dim = seq_dim
        return _gather_along_seq_dim(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_along_seq_dim(g, ctx.seq_dim), None


class _ScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        ctx.seq_dim = seq_dim
        return _split_along_seq_dim(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _gather_along_seq_dim(g, ctx.seq_dim), None


class _CopyToExpertMP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tokens_per_expert):
        ctx.tpe = tokens_per_expert
        return _dmoe_slice(x, tokens_per_expert)

    @staticmethod
    def backward(ctx, g):
        return _dmoe_gather(g, ctx.tpe), None


class _GatherFromExpertMP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tokens_per_expert):
        ctx.tpe = tokens_per_expert
        return _dmoe_gather(x, tokens_per_expert)

    @staticmethod
    def backward(ctx, g):
        return _dmoe_slice(g, ctx.tpe), None


def copy_to_model_parallel_region(x):
    return _CopyToMP.apply(x)


def reduce_from_model_parallel_region(x):
    return _ReduceFromMP.apply(x)


def scatter_to_model_parallel_region(x):
    return _ScatterToMP.apply(x)


def gather_from_model_parallel_region(x):
    return _GatherFromMP.apply(x)


def reduce_scatter_to_sequence_parallel_region(x, seq_dim=0):
    return _ReduceScatterToSP.apply(x, seq_dim)


def gather_from_sequence_parallel_region(x, seq_dim=0):
    return _GatherFromSP.apply(x, seq_dim)


def scatter_to_sequence_parallel_region(x, seq_dim=1):
    return _ScatterToSP.apply(x, seq_dim)


def copy_to_expert_model_parallel_region(x, tokens_per_expert):
    return _CopyToExpertMP.apply(x, tokens_per_expert)


def gather_from_expert_model_parallel_region(x, tokens_per_expert):
    return _GatherFromExpertMP.apply(x, tokens_per_expert)
