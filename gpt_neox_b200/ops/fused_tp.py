"""Tensor + sequence parallel linear layers whose collective is fused into the GEMM kernel.

  ag_linear      y = all_gather_rows(x_shard) @ W^T + b          (column-parallel forward,
                 megatron/mpu/layers.py:567-576); backward = GEMM -> reduce-scatter of dX
  linear_rs      y_shard = reduce_scatter_rows(x @ W^T) + b + r   (row-parallel forward,
                 megatron/mpu/layers.py:773-779); backward = all-gather -> GEMM
  linear_ar      y = all_reduce(x @ W^T) + b                      (row-parallel forward without sequence
                 parallelism): reduce-scatter in the GEMM epilogue, owners store the reduced rows to all ranks
  mlp_gelu_sp    the whole MLP of a block, all-gather in front of the first GEMM and the block's
                 single reduce-scatter (GPT-J residual: attention partial sums ride along as a
                 residual of the second GEMM, megatron/model/transformer.py:1116) behind the second
The kernels push tiles / shards into peer memory over NVLink from inside the GEMM
(csrc/gemm_tcgen05.cu, modes COMM_AG / COMM_RS); this module only arranges operands and autograd.
"""
from __future__ import annotations

import torch

from ..comm import collectives, symm
from . import _lib
from .elementwise import bias_grad, colsum
from .gemm import wgrad


def backend(x, group):
    """The symmetric-memory backend of ``group`` if the fused path can serve ``x``."""
    if collectives.get_mode() != "fused" or not x.is_cuda or x.dtype not in _lib.H16:
        return None
    return symm.backend_for(group)


def _keeps(ctx) -> bool:
    """Ask for a pool slot only when a backward pass will come for it (the input gradient's fused reduce-scatter is
    what makes the release safe, the weight gradient is what reads the slot).  Under pipeline parallelism, where the
    forward passes of later micro-batches run between the backward passes of earlier ones, the gathered operand is
    copied as before: the pooled form has only been run with one micro-batch in flight."""
    from .. import parallel as mpu
    return bool(ctx.needs_input_grad[0] and ctx.needs_input_grad[1] and mpu.get_pipe_parallel_world_size() == 1)


def _release(ctx):
    """Give the gather slot of this node back.  A second backward pass over the same graph (``retain_graph``) would
    read a slot that has been reused: the pooled form is for the single backward pass of training."""
    slot, ctx.slot = getattr(ctx, "slot", None), None
    if slot is not None:
        ctx.be.pool_release(slot)


def _rows(x):
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.is_contiguous() else x2.contiguous()


class _AGLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, b, be):
        x2 = _rows(x_shard)
        # the gathered operand is needed again by the weight-gradient GEMM: it stays in a pool slot of the symmetric
        # workspace when one is free, else it is copied out of the two-deep gather ring
        y, gathered, slot = be.ag_gemm(x2, w, bias=b, keep=_keeps(ctx))
        ctx.save_for_backward(gathered if (slot is not None or not any(ctx.needs_input_grad)) else gathered.clone(), w)
        ctx.be, ctx.has_bias, ctx.in_shape, ctx.slot, ctx.bias = be, b is not None, x_shard.shape, slot, b
        return y.view(x_shard.shape[0] * be.ws, *x_shard.shape[1:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        xf, w = ctx.saved_tensors
        gy2 = _rows(gy)
        dw = wgrad(gy2, xf, w) if ctx.needs_input_grad[1] else None
        _release(ctx)                  # after the last read of the slot, before the fused call below
        dx = ctx.be.gemm_rs(gy2, w, trans_b=True).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        db = bias_grad(gy2, ctx.bias) if ctx.has_bias else None
        return dx, dw, db, None


class _LinearRSFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, res_shard, be):
        x2 = _rows(x)
        r2 = _rows(res_shard) if res_shard is not None else None
        y = be.gemm_rs(x2, w, bias=b, residual2=r2)
        ctx.save_for_backward(x2, w)
        ctx.be, ctx.has_bias, ctx.has_res, ctx.bias = be, b is not None, res_shard is not None, b
        ctx.x_shape = x.shape
        return y.view(x.shape[0] // be.ws, *x.shape[1:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = _rows(gy)
        dx, g_full = ctx.be.ag_gemm(g2, w, trans_b=True)          # dX = all_gather(g) @ W
        dw = wgrad(g_full, x2, w) if ctx.needs_input_grad[1] else None
        db = bias_grad(g2, ctx.bias) if ctx.has_bias else None    # partial over this rank's rows: the
        return dx.view(ctx.x_shape), dw, db, (gy if ctx.has_res else None), None  # engine sums it over TP


class _MLPGeluSPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w1, b1, w2, partial_full, bias_total, res_shard, kind, be):
        x2 = _rows(x_shard)
        m = x2.shape[0] * be.ws
        pre = torch.empty((m, w1.shape[0]), device=x2.device, dtype=x2.dtype)
        h, gathered, slot = be.ag_gemm(x2, w1, bias=b1, gelu=kind, aux_out=pre, aux_deriv=True,     # pre = gelu'(.)
                                       keep=_keeps(ctx))
        xf = gathered if (slot is not None or not any(ctx.needs_input_grad)) else gathered.clone()
        ctx.slot = slot
        pf = _rows(partial_full) if partial_full is not None else None
        rs = _rows(res_shard) if res_shard is not None else None
        out = be.gemm_rs(h, w2, residual=pf, bias=bias_total, residual2=rs)
        ctx.save_for_backward(xf, w1, w2, pre, h)
        ctx.be, ctx.kind = be, kind
        ctx.flags = (b1 is not None, partial_full is not None, bias_total is not None, res_shard is not None)
        ctx.bias1 = b1
        ctx.in_shape = x_shard.shape
        ctx.pf_shape = partial_full.shape if partial_full is not None else None
        return out.view(x_shard.shape[:-1] + (w2.shape[0],))

    @staticmethod
    def backward(ctx, g):
        xf, w1, w2, pre, h = ctx.saved_tensors
        has_b1, has_pf, has_bt, has_rs = ctx.flags
        be = ctx.be
        g2 = _rows(g)
        # d(pre) = (all_gather(g) @ W2) * gelu'(pre): gather fused in front, derivative in the epilogue
        dpre, g_full = be.ag_gemm(g2, w2, trans_b=True, dgelu_aux=pre, dgelu="mul")
        dw2 = wgrad(g_full, h, w2) if ctx.needs_input_grad[3] else None
        d_pf = g_full.clone().view(ctx.pf_shape) if has_pf else None
        # every rank adds bias_total to its own rows only; its gradient over ALL rows, divided by the
        # number of ranks that will each report it, keeps the sum over ranks exact
        d_bt = (colsum(g_full, torch.float32) / be.ws).to(g.dtype) if has_bt else None
        dw1 = wgrad(dpre, xf, w1) if ctx.needs_input_grad[1] else None
        _release(ctx)                  # after the last read of the slot, before the fused call below
        dx = be.gemm_rs(dpre, w1, trans_b=True).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        db1 = bias_grad(dpre, ctx.bias1) if has_b1 else None
        return dx, dw1, db1, dw2, d_pf, d_bt, (g if has_rs else None), None, None


class _LinearARFn(torch.autograd.Function):
    """Row-parallel linear without sequence parallelism: y = all_reduce(x @ W^T) + b with the reduction
    inside the GEMM kernel (megatron/mpu/layers.py:773-779, mappings.py:31-50).  Backward needs no
    collective: the incoming gradient is replicated."""

    @staticmethod
    def forward(ctx, x, w, b, be):
        x2 = _rows(x)
        y = be.gemm_ar(x2, w, bias=b).clone()
        ctx.save_for_backward(x2, w)
        ctx.has_bias, ctx.x_shape, ctx.bias = b is not None, x.shape, b
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        from .gemm import gemm
        x2, w = ctx.saved_tensors
        g2 = _rows(gy)
        dx = gemm(g2, w, trans_b=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = wgrad(g2, x2, w) if ctx.needs_input_grad[1] else None
        db = bias_grad(g2, ctx.bias) if ctx.has_bias else None
        return dx, dw, db, None


def linear_ar(x, w, b, be):
    return _LinearARFn.apply(x, w, b, be)


def ag_linear(x_shard, w, b, be):
    return _AGLinearFn.apply(x_shard, w, b, be)


def linear_rs(x, w, b, res_shard, be):
    return _LinearRSFn.apply(x, w, b, res_shard, be)


def mlp_gelu_sp(x_shard, w1, b1, w2, partial_full, bias_total, res_shard, kind, be):
    return _MLPGeluSPFn.apply(x_shard, w1, b1, w2, partial_full, bias_total, res_shard, kind, be)
