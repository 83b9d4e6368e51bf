"""LayerNorm / RMSNorm with fp32 statistics.

CUDA bf16 tensors run ``nx_norm_fwd`` / ``nx_norm_bwd`` (csrc/norm.cu); everything else runs the
PyTorch statement of the same math (megatron/model/norms.py:62-99 for RMSNorm,
``torch.nn.LayerNorm`` for LayerNorm), which is also the oracle in the tests.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import LAUNCHES

LN, RMS = 0, 1


def _cuda_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


def _accum_param_grad(param: torch.Tensor, g_f32: torch.Tensor):
    """Route a fp32 parameter gradient: into ``main_grad`` if the engine installed one."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        mg.add_(g_f32.view_as(mg))
        return None
    return g_f32.to(param.dtype)


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, kind, x, gamma, beta, eps, gamma2, beta2):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y1 = torch.empty_like(x2)
        dual = gamma2 is not None
        y2 = torch.empty_like(x2) if dual else None
        mean = torch.empty(rows, device=x.device, dtype=torch.float32) if kind == LN else None
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib().nx_norm_fwd(
            kind, _lib.ptr(x2), _lib.ptr(gamma), _lib.ptr(beta), _lib.ptr(y1), _lib.ptr(gamma2),
            _lib.ptr(beta2), _lib.ptr(y2), _lib.ptr(mean), _lib.ptr(rstd), rows, H, float(eps),
            _lib.stream()), "nx_norm_fwd")
        ctx.kind, ctx.dual, ctx.shape = kind, dual, x.shape
        ctx.has_beta = beta is not None
        ctx.has_beta2 = beta2 is not None
        ctx.save_for_backward(x2, gamma, gamma2, mean, rstd)
        if dual:
            return y1.view(x.shape), y2.view(x.shape)
        return y1.view(x.shape)

    @staticmethod
    def backward(ctx, *gys):
        x2, gamma, gamma2, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        L = _lib.lib()
        blocks = L.nx_norm_bwd_blocks(rows)
        ws = torch.empty(blocks * 2 * H, device=x2.device, dtype=torch.float32)
        dx = torch.empty_like(x2)
        outs = []
        dx_in = None
        for gy, g, has_b in ((gys[0], gamma, ctx.has_beta),
                             (gys[1] if ctx.dual else None, gamma2, ctx.has_beta2)):
            if g is None:
                continue
            if gy is None:
                outs.append((None, None))
                continue
            gy2 = gy.reshape(rows, H)
            if not gy2.is_contiguous():
                gy2 = gy2.contiguous()
            dg = torch.empty(H, device=x2.device, dtype=torch.float32)
            db = torch.empty(H, device=x2.device, dtype=torch.float32) if has_b else None
            LAUNCHES["n"] += 2
            _lib.check(L.nx_norm_bwd(
                ctx.kind, _lib.ptr(gy2), _lib.ptr(x2), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(g),
                _lib.ptr(dx_in), _lib.ptr(dx), _lib.ptr(dg), _lib.ptr(db), _lib.ptr(ws), rows, H, 0,
                _lib.stream()), "nx_norm_bwd")
            dx_in = dx  # the second norm of a dual pair adds onto the first one's dx
            outs.append((dg, db))
        return (None, dx.view(ctx.shape) if dx_in is not None else None,
                outs[0][0], outs[0][1], None,
                outs[1][0] if ctx.dual else None, outs[1][1] if ctx.dual else None)


class _ParamGrad(torch.autograd.Function):
    """Identity on a parameter whose backward converts the fp32 kernel gradient to the
    parameter's dtype (or accumulates it into ``param.main_grad``)."""

    @staticmethod
    def forward(ctx, p):
        ctx.p = p
        return p.detach()

    @staticmethod
    def backward(ctx, g):
        return _accum_param_grad(ctx.p, g)


def _wrap(p):
    return None if p is None else (_ParamGrad.apply(p) if p.requires_grad else p)


def layer_norm(x, weight, bias=None, eps: float = 1e-5):
    if _cuda_ok(x):
        return _NormFn.apply(LN, x, _wrap(weight), _wrap(bias), eps, None, None)
    if x.is_cuda:
        raise _lib.KernelError(f"layer_norm: CUDA path needs bf16 and H % 8 == 0, got {x.dtype} {tuple(x.shape)}")
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def dual_layer_norm(x, w1, b1, w2, b2, eps: float = 1e-5):
    """Two LayerNorms of the same input from one pass (GPT-J parallel residual,
    megatron/model/transformer.py:1083)."""
    if _cuda_ok(x):
        return _NormFn.apply(LN, x, _wrap(w1), _wrap(b1), eps, _wrap(w2), _wrap(b2))
    return layer_norm(x, w1, b1, eps), layer_norm(x, w2, b2, eps)


def rms_norm(x, weight, eps: float = 1e-8):
    if _cuda_ok(x):
        return _NormFn.apply(RMS, x, _wrap(weight), None, eps, None, None)
    if x.is_cuda:
        raise _lib.KernelError(f"rms_norm: CUDA path needs bf16 and H % 8 == 0, got {x.dtype}")
    dtype = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (weight.float() * (xf * torch.rsqrt(var + eps))).to(dtype)


def dual_rms_norm(x, w1, w2, eps: float = 1e-8):
    if _cuda_ok(x):
        return _NormFn.apply(RMS, x, _wrap(w1), None, eps, _wrap(w2), None)
    return rms_norm(x, w1, eps), rms_norm(x, w2, eps)
