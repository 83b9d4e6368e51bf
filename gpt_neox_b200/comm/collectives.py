"""Collective entry points used by the parallel layers.

Every function has a torch.distributed implementation (the ``nccl_baseline`` mode of the
framework, and the only one on CPU / gloo).  In ``fused`` mode on CUDA the all-reduce /
all-gather / reduce-scatter of bf16 / fp32 tensors are served by this library's own NVLink
kernels over symmetric memory (``comm.symm``) when a symmetric workspace exists for the group.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_MODE = {"mode": "nccl_baseline"}
#: bytes moved by collectives issued through this module since the last reset (comms logging)
STATS = {"all_reduce": [0, 0], "all_gather": [0, 0], "reduce_scatter": [0, 0], "broadcast": [0, 0]}


def set_mode(mode: str):
    assert mode in ("fused", "nccl_baseline")
    _MODE["mode"] = mode


def get_mode() -> str:
    return _MODE["mode"]


_OBSERVER = None          # a comms logger (obs.profiling.CommsLogger) timing the NVLink collectives below


def set_observer(obs):
    global _OBSERVER
    _OBSERVER = obs


def _own(op, x, nbytes, group, call):
    """Run one of this library's own collectives, timed when a comms logger is installed."""
    if _OBSERVER is None:
        return call()
    with _OBSERVER.observe(op + "[nvlink]", nbytes, dist.get_world_size(group), cuda=x.is_cuda):
        return call()


def _log(kind, t):
    s = STATS[kind]
    s[0] += 1
    s[1] += t.numel() * t.element_size()


def _fused_backend(x, group):
    if _MODE["mode"] != "fused" or not x.is_cuda:
        return None
    from . import symm
    return symm.backend_for(group)


def all_reduce(x: torch.Tensor, group=None, op=dist.ReduceOp.SUM) -> torch.Tensor:
    """In-place sum (or ``op``) over ``group``; returns ``x``."""
    _log("all_reduce", x)
    be = _fused_backend(x, group) if op == dist.ReduceOp.SUM else None
    if be is not None and be.supports(x):
        return _own("all_reduce", x, x.numel() * x.element_size(), group, lambda: be.all_reduce(x))
    dist.all_reduce(x, op=op, group=group)
    return x


def all_gather_list(x: torch.Tensor, group=None) -> list:
    ws = dist.get_world_size(group)
    _log("all_gather", x)
    parts = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(parts, x, group=group)
    return parts


def all_gather_dim(x: torch.Tensor, dim: int, group=None) -> torch.Tensor:
    """Concatenate every rank's ``x`` along ``dim``."""
    ws = dist.get_world_size(group)
    _log("all_gather", x)
    x = x.contiguous()
    be = _fused_backend(x, group)
    if dim == 0:
        if be is not None and be.supports(x):
            return _own("all_gather", x, ws * x.numel() * x.element_size(), group, lambda: be.all_gather0(x))
        out = torch.empty((ws * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    parts = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=dim).contiguous()


def reduce_scatter_dim(x: torch.Tensor, dim: int, group=None) -> torch.Tensor:
    """Sum over ranks, rank r keeps chunk r of ``dim``."""
    ws = dist.get_world_size(group)
    _log("reduce_scatter", x)
    be = _fused_backend(x, group)
    if dim == 0:
        x = x.contiguous()
        if be is not None and be.supports(x):
            return _own("reduce_scatter", x, x.numel() * x.element_size(), group, lambda: be.reduce_scatter0(x))
        out = torch.empty((x.shape[0] // ws,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.reduce_scatter_tensor(out, x, group=group)
        else:  # gloo has no reduce_scatter: all-reduce then slice
            y = x.clone()
            dist.all_reduce(y, group=group)
            out.copy_(y.chunk(ws, dim=0)[dist.get_rank(group)])
        return out
    chunks = [c.contiguous() for c in x.chunk(ws, dim=dim)]
    out = torch.empty_like(chunks[0])
    if x.is_cuda:
        dist.reduce_scatter(out, chunks, group=group)
    else:
        y = x.clone()
        dist.all_reduce(y, group=group)
        out.copy_(y.chunk(ws, dim=dim)[dist.get_rank(group)])
    return out


def broadcast(x: torch.Tensor, src: int, group=None) -> torch.Tensor:
    _log("broadcast", x)
    dist.broadcast(x, src, group=group)
    return x
