"""RWKV-6 WKV operator (csrc/wkv6.cu): chunk-parallel linear recurrence with data-dependent decay.

``r, k, v, w``: ``[batch, time, heads * N]`` views with contiguous channels (time-major memory is fine);
``u``: ``[heads, N]``.  ``w`` is the log-log decay: the per-step decay is ``exp(-exp(w))``.
Reference: ``WKV`` autograd function, megatron/model/rwkv/v6/rwkv.py:12-97.
"""
from __future__ import annotations

import torch

from . import _lib
from .gemm import LAUNCHES


def wkv6_reference(r, k, v, w, u):
    """Sequential fp32 statement. Returns y [b, t, c] in the dtype of ``r``."""
    B, T, C = r.shape
    H, N = u.shape
    dt = r.dtype
    r, k, v = (x.float().reshape(B, T, H, N) for x in (r, k, v))
    d = torch.exp(-torch.exp(w.float())).reshape(B, T, H, N)
    uf = u.float()
    S = r.new_zeros(B, H, N, N)
    ys = []
    for t in range(T):
        kv = k[:, t, :, :, None] * v[:, t, :, None, :]
        ys.append(torch.einsum("bhi,bhij->bhj", r[:, t], uf[None, :, :, None] * kv + S))
        S = d[:, t, :, :, None] * S + kv
    return torch.stack(ys, 1).reshape(B, T, C).to(dt)


def decay_grad_from_gr_gk(r, k, v, w, u, gy, gr, gk):
    """dL/dw from gr and gk: with Q_t[i] = sum_j dL/dS_t[i][j] * S_t[i][j] one has
    Q_{t-1} - Q_t = r_t gr_t - k_t gk_t and  dL/d(ew_t) = Q_t - k_t (gk_t - r_t u <gy_t, v_t>)."""
    B, T, C = r.shape
    H, N = u.shape
    f = lambda x: x.float().reshape(B, T, H, N)
    r_, k_, v_, gy_, gr_, gk_ = f(r), f(k), f(v), f(gy), f(gr), f(gk)
    s = (gy_ * v_).sum(-1, keepdim=True)
    delta = r_ * gr_ - k_ * gk_
    Q = delta.flip(1).cumsum(1).flip(1) - delta              # exclusive reverse cumulative sum
    g_ew = Q - k_ * (gk_ - r_ * u.float()[None, None] * s)
    ew = -torch.exp(w.float()).reshape(B, T, H, N)
    gw = (g_ew * ew).reshape(B, T, C)
    gu = (r_ * k_ * s).sum((0, 1))
    return gw, gu


def _pass(mode, a, b, c, w, u, out, local, start, sumew, B, T, H, N):
    LAUNCHES["n"] += 1
    o = (out.stride(0), out.stride(1), int(out.dtype == torch.float32)) if out is not None else (0, 0, 0)
    _lib.check(_lib.lib(b).nx_wkv6_pass(mode, _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.ptr(w), b.stride(0),
                                       b.stride(1), _lib.ptr(u), _lib.ptr(out), o[0], o[1], o[2], _lib.ptr(local),
                                       _lib.ptr(start), _lib.ptr(sumew), B, T, H, N, _lib.stream()), "nx_wkv6_pass")


def _same_layout(*ts):
    """Views sharing (batch, time) strides with contiguous channels; copies to time-major otherwise."""
    s0 = (ts[0].stride(0), ts[0].stride(1))
    if all(t.stride(2) == 1 and (t.stride(0), t.stride(1)) == s0 for t in ts):
        return ts
    B, T, C = ts[0].shape
    out = []
    for t in ts:
        buf = torch.empty((T, B, C), device=t.device, dtype=t.dtype).transpose(0, 1)
        buf.copy_(t)
        out.append(buf)
    return tuple(out)


class _WkvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, k, v, w, u):
        B, T, C = r.shape
        H, N = u.shape
        r, k, v, w = _same_layout(r, k, v, w)
        u32 = u.float().contiguous()
        nc = _lib.lib().nx_wkv6_chunks(T)
        dev = r.device
        local = torch.empty((B, H, nc, N, N), device=dev, dtype=torch.float32)
        start = torch.empty_like(local)
        sumew = torch.empty((B, H, nc, N), device=dev, dtype=torch.float32)
        y = torch.empty((T, B, C), device=dev, dtype=r.dtype).transpose(0, 1)
        _pass(0, None, k, v, w, u32, None, local, start, sumew, B, T, H, N)
        _pass(2, None, k, v, w, u32, None, local, start, sumew, B, T, H, N)
        _pass(4, r, k, v, w, u32, y, local, start, sumew, B, T, H, N)
        ctx.save_for_backward(r, k, v, w, u32, start, sumew)
        ctx.u_dtype = u.dtype
        return y

    @staticmethod
    def backward(ctx, gy):
        r, k, v, w, u32, start, sumew = ctx.saved_tensors
        B, T, C = r.shape
        H, N = u32.shape
        if gy.stride(2) != 1 or (gy.stride(0), gy.stride(1)) != (r.stride(0), r.stride(1)):
            buf = torch.empty((T, B, C), device=gy.device, dtype=gy.dtype).transpose(0, 1)
            buf.copy_(gy)
            if (buf.stride(0), buf.stride(1)) != (r.stride(0), r.stride(1)):
                r, k, v, w = (x.contiguous() for x in (r, k, v, w))
                buf = gy.contiguous()
            gy = buf
        dev = r.device
        f32 = lambda: torch.empty((T, B, C), device=dev, dtype=torch.float32).transpose(0, 1)
        gr, gk, gv = f32(), f32(), f32()
        # forward-state sweep: gr (start states were kept from the forward)
        _pass(6, gy, k, v, w, u32, gr, None, start, sumew, B, T, H, N)
        # reverse state G: local, fold, then gk (rows) and gv (columns)
        local = torch.empty_like(start)
        rstart = torch.empty_like(start)
        _pass(1, None, r, gy, w, u32, None, local, rstart, sumew, B, T, H, N)
        _pass(3, None, r, gy, w, u32, None, local, rstart, sumew, B, T, H, N)
        _pass(7, v, r, gy, w, u32, gk, None, rstart, sumew, B, T, H, N)
        _pass(5, k, r, gy, w, u32, gv, None, rstart, sumew, B, T, H, N)
        gw, gu = decay_grad_from_gr_gk(r, k, v, w, u32, gy, gr, gk)
        dt = r.dtype
        return gr.to(dt), gk.to(dt), gv.to(dt), gw.to(dt), gu.to(ctx.u_dtype)


def wkv6(r, k, v, w, u):
    """y [b, t, c] of the RWKV-6 recurrence; differentiable in all five arguments."""
    if r.is_cuda:
        if r.dtype not in _lib.H16 or u.shape[1] not in (32, 64):
            raise _lib.KernelError("wkv6: CUDA path needs bf16 and head size 32 or 64")
        return _WkvFn.apply(r, k, v, w, u)
    return wkv6_reference(r, k, v, w, u)
