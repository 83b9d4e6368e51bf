"""Mamba-1 operators: causal depthwise conv1d + SiLU and the S6 selective scan (csrc/mamba.cu).

Every tensor is ``[batch, time, channel]`` *logically* and may be any strided view with a contiguous
channel dimension, so ``[seq, batch, channel]`` activations are passed as ``x.transpose(0, 1)`` without a
copy.  The CPU path is the plain PyTorch statement of the same recurrences (the oracle of the GPU tests);
on CUDA the kernels always run.  Reference call sites: megatron/model/mamba/mamba.py:220-247,264-320.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import LAUNCHES


def _btd(t):
    assert t.dim() == 3 and t.stride(2) == 1, "expected [batch, time, channel] with contiguous channels"
    return t


# ------------------------------------------------------------------------------------------ conv1d
def causal_conv1d_silu_reference(x, weight, bias):
    """x [b, l, d]; weight [d, w]; bias [d] or None -> silu(causal depthwise conv)."""
    w = weight.shape[1]
    xt = x.transpose(1, 2).float()
    y = F.conv1d(xt, weight.float().unsqueeze(1), None if bias is None else bias.float(), padding=w - 1,
                 groups=weight.shape[0])[..., : x.shape[1]]
    return F.silu(y).transpose(1, 2).to(x.dtype)


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        B, L, D = x.shape
        y = torch.empty((L, B, D), device=x.device, dtype=x.dtype).transpose(0, 1)   # time-major memory
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x).nx_conv1d_silu_fwd(_lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(weight),
                                                 _lib.ptr(bias), _lib.ptr(y), y.stride(0), y.stride(1), B, L, D,
                                                 weight.shape[1], _lib.stream()), "nx_conv1d_silu_fwd")
        ctx.save_for_backward(x, weight, bias)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight, bias = ctx.saved_tensors
        B, L, D = x.shape
        if gy.stride(2) != 1:
            gy = gy.contiguous()
        dx = torch.empty((L, B, D), device=x.device, dtype=x.dtype).transpose(0, 1)
        dw = torch.zeros(weight.shape, device=x.device, dtype=torch.float32)
        db = torch.zeros(D, device=x.device, dtype=torch.float32) if bias is not None else None
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x).nx_conv1d_silu_bwd(_lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(weight),
                                                 _lib.ptr(bias), _lib.ptr(gy), gy.stride(0), gy.stride(1),
                                                 _lib.ptr(dx), dx.stride(0), dx.stride(1), _lib.ptr(dw),
                                                 _lib.ptr(db), B, L, D, weight.shape[1], _lib.stream()),
                   "nx_conv1d_silu_bwd")
        return dx, dw.to(weight.dtype), None if db is None else db.to(bias.dtype)


def causal_conv1d_silu(x, weight, bias=None):
    """``silu(depthwise_causal_conv(x))`` for x [b, l, d] (strided ok), weight [d, w<=4], bias [d]."""
    _btd(x)
    if x.is_cuda:
        if x.dtype not in _lib.H16 or weight.shape[1] > 4:
            raise _lib.KernelError("causal_conv1d_silu: CUDA path needs bf16 and kernel width <= 4")
        return _ConvFn.apply(x, weight.contiguous(), None if bias is None else bias.contiguous())
    return causal_conv1d_silu_reference(x, weight, bias)


# ------------------------------------------------------------------------------------------ scan
def selective_scan_reference(x, dt, A, Bm, Cm, D=None, z=None, dt_bias=None):
    """Sequential fp32 statement of the S6 recurrence. x, dt, z [b, l, d]; A [d, n]; Bm, Cm [b, l, n]."""
    dtype = x.dtype
    x, dt, Bm, Cm = x.float(), dt.float(), Bm.float(), Cm.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    dt = F.softplus(dt)
    b, l, d = x.shape
    h = x.new_zeros(b, d, A.shape[1])
    ys = []
    for t in range(l):
        a = torch.exp(dt[:, t, :, None] * A[None].float())
        h = a * h + dt[:, t, :, None] * Bm[:, t, None, :] * x[:, t, :, None]
        ys.append((h * Cm[:, t, None, :]).sum(-1))
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + D.float() * x
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(dtype)


class _ScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A, Bm, Cm, D, z, dt_bias):
        L_ = _lib.lib(x)
        B, L, Dm = x.shape
        dev = x.device
        nc = L_.nx_scan_chunks(L)
        out = torch.empty((L, B, Dm), device=dev, dtype=x.dtype).transpose(0, 1)   # time-major memory
        state = torch.empty((B, nc, Dm, 16), device=dev, dtype=torch.float32)
        h0 = torch.empty((B, nc, Dm, 16), device=dev, dtype=torch.float32)
        sumdt = torch.empty((B, nc, Dm), device=dev, dtype=torch.float32)
        zs = (z.stride(0), z.stride(1)) if z is not None else (0, 0)
        LAUNCHES["n"] += 2 if nc > 1 else 1
        _lib.check(L_.nx_selective_scan_fwd(
            _lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(dt), dt.stride(0), dt.stride(1), _lib.ptr(z), zs[0],
            zs[1], _lib.ptr(Bm), Bm.stride(0), Bm.stride(1), _lib.ptr(Cm), Cm.stride(0), Cm.stride(1),
            _lib.ptr(A), _lib.ptr(D), _lib.ptr(dt_bias), _lib.ptr(out), out.stride(0), out.stride(1),
            _lib.ptr(state), _lib.ptr(sumdt), _lib.ptr(h0), B, L, Dm, _lib.stream()), "nx_selective_scan_fwd")
        ctx.save_for_backward(x, dt, A, Bm, Cm, D, z, dt_bias, sumdt, h0)
        return out

    @staticmethod
    def backward(ctx, gout):
        x, dt, A, Bm, Cm, D, z, dt_bias, sumdt, h0 = ctx.saved_tensors
        L_ = _lib.lib(x)
        B, L, Dm = x.shape
        dev = x.device
        if gout.stride(2) != 1:
            gout = gout.contiguous()
        nc = L_.nx_scan_chunks(L)
        nb = L_.nx_scan_channel_blocks(Dm)
        dx = torch.empty((L, B, Dm), device=dev, dtype=x.dtype).transpose(0, 1)
        ddt = torch.empty((L, B, Dm), device=dev, dtype=x.dtype).transpose(0, 1)
        dz = torch.empty((L, B, Dm), device=dev, dtype=x.dtype).transpose(0, 1) if z is not None else None
        part = torch.empty((nb, B, L, 32), device=dev, dtype=torch.float32)
        dA = torch.zeros((Dm, 16), device=dev, dtype=torch.float32)
        dD = torch.zeros(Dm, device=dev, dtype=torch.float32) if D is not None else None
        dbias = torch.zeros(Dm, device=dev, dtype=torch.float32)
        E = torch.empty((B, nc, Dm, 16), device=dev, dtype=torch.float32)
        zs = (z.stride(0), z.stride(1)) if z is not None else (0, 0)
        LAUNCHES["n"] += 2 if nc > 1 else 1
        _lib.check(L_.nx_selective_scan_bwd(
            _lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(dt), dt.stride(0), dt.stride(1), _lib.ptr(z), zs[0],
            zs[1], _lib.ptr(Bm), Bm.stride(0), Bm.stride(1), _lib.ptr(Cm), Cm.stride(0), Cm.stride(1),
            _lib.ptr(A), _lib.ptr(D), _lib.ptr(dt_bias), _lib.ptr(gout), gout.stride(0), gout.stride(1),
            _lib.ptr(dx), _lib.ptr(ddt), _lib.ptr(dz), dx.stride(0), dx.stride(1), _lib.ptr(part), _lib.ptr(dA),
            _lib.ptr(dD), _lib.ptr(dbias), _lib.ptr(sumdt), _lib.ptr(h0), _lib.ptr(E), B, L, Dm, _lib.stream()),
            "nx_selective_scan_bwd")
        bc = part.sum(0)
        dB = bc[..., :16].to(Bm.dtype)
        dC = bc[..., 16:].to(Cm.dtype)
        return dx, ddt, dA, dB, dC, dD, dz, dbias


def selective_scan(x, dt, A, Bm, Cm, D=None, z=None, dt_bias=None):
    """``y = (scan(x; softplus(dt + dt_bias), A, B, C) + D x) * silu(z)``.

    x, dt, z: [b, l, d] bf16 views with contiguous channels; A [d, 16] fp32 (negative); Bm, Cm [b, l, 16];
    D, dt_bias [d] fp32."""
    _btd(x), _btd(dt), _btd(Bm), _btd(Cm)
    if x.is_cuda:
        if x.dtype not in _lib.H16 or A.shape[1] != 16:
            raise _lib.KernelError("selective_scan: CUDA path needs bf16 activations and d_state == 16")
        if dt_bias is None:
            dt_bias = torch.zeros(x.shape[2], device=x.device, dtype=torch.float32)
        return _ScanFn.apply(x, dt, A.float().contiguous(), Bm, Cm, None if D is None else D.float().contiguous(),
                             z, dt_bias.float().contiguous())
    return selective_scan_reference(x, dt, A, Bm, Cm, D, z, dt_bias)
