"""Scaled causal / masked softmax (the non-flash attention path).

Module-level parity with the reference's ``scaled_upper_triang_masked_softmax_cuda`` and
``scaled_masked_softmax_cuda`` extensions (megatron/model/fused_softmax.py:24-83): the same
``forward`` / ``backward`` pairs, exposed as autograd functions. CUDA bf16 -> csrc/softmax.cu,
otherwise PyTorch.
"""
from __future__ import annotations

import torch

from . import _lib
from .gemm import LAUNCHES


def _cuda_ok(x):
    return x.is_cuda and x.dtype in _lib.H16


class _CausalSoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        assert x.dim() == 3
        xc = x.contiguous()
        y = torch.empty_like(xc)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(xc).nx_softmax_causal_fwd(_lib.ptr(xc), _lib.ptr(y), xc.shape[0], xc.shape[1],
                                                    xc.shape[2], float(scale), _lib.stream()),
                   "nx_softmax_causal_fwd")
        ctx.scale = scale
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, gy):
        (y,) = ctx.saved_tensors
        gyc = gy.contiguous()
        dx = torch.empty_like(y)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(gyc).nx_softmax_bwd(_lib.ptr(gyc), _lib.ptr(y), _lib.ptr(dx),
                                             y.shape[0] * y.shape[1], y.shape[2], float(ctx.scale),
                                             _lib.stream()), "nx_softmax_bwd")
        return dx, None


class _MaskedSoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, scale):
        assert x.dim() == 4
        xc = x.contiguous()
        b, np_, sq, sk = xc.shape
        m = None
        mb = 1
        if mask is not None:
            m = mask.to(torch.uint8).contiguous()
            mb = m.shape[0]
        y = torch.empty_like(xc)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(xc).nx_softmax_masked_fwd(_lib.ptr(xc), _lib.ptr(m), _lib.ptr(y), b, np_, sq, sk,
                                                    mb, float(scale), _lib.stream()),
                   "nx_softmax_masked_fwd")
        ctx.scale = scale
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, gy):
        (y,) = ctx.saved_tensors
        gyc = gy.contiguous()
        dx = torch.empty_like(y)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(gyc).nx_softmax_bwd(_lib.ptr(gyc), _lib.ptr(y), _lib.ptr(dx),
                                             y.numel() // y.shape[-1], y.shape[-1], float(ctx.scale),
                                             _lib.stream()), "nx_softmax_bwd")
        return dx, None, None


def scaled_causal_softmax(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """x: [attn_batches, sq, sk]; row i attends to columns <= i + (sk - sq); masked probs are 0."""
    if _cuda_ok(x):
        return _CausalSoftmaxFn.apply(x, scale)
    if x.is_cuda:
        raise _lib.KernelError("scaled_causal_softmax: CUDA path needs bf16")
    sq, sk = x.shape[-2], x.shape[-1]
    keep = torch.ones(sq, sk, dtype=torch.bool, device=x.device).tril(diagonal=sk - sq)
    xf = (x.float() * scale).masked_fill(~keep, float("-inf"))
    return torch.softmax(xf, dim=-1).masked_fill(~keep, 0.0).to(x.dtype)


def scaled_masked_softmax(x: torch.Tensor, mask: torch.Tensor | None, scale: float = 1.0) -> torch.Tensor:
    """x: [b, np, sq, sk]; mask: [b|1, 1, sq, sk], True/1 = masked (filled with -10000)."""
    if _cuda_ok(x):
        return _MaskedSoftmaxFn.apply(x, mask, scale)
    if x.is_cuda:
        raise _lib.KernelError("scaled_masked_softmax: CUDA path needs bf16")
    xf = x.float() * scale
    if mask is not None:
        xf = xf.masked_fill(mask.bool(), -10000.0)
    return torch.softmax(xf, dim=-1).to(x.dtype)


def get_batch_per_block(sq: int, sk: int, b: int, np_: int) -> int:
    """Same contract as ``scaled_masked_softmax_cuda.get_batch_per_block``
    (megatron/fused_kernels/scaled_masked_softmax.h:338-352)."""
    p2 = 1
    while p2 < sk:
        p2 <<= 1
    warp = min(p2, 32)
    return (128 // warp) * (2 if p2 <= 128 else 1)
