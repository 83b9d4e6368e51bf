"""Rotary position embedding, full or partial, applied to strided q / k views.

Convention of megatron/model/positional_embeddings.py:38-127 (rotate-half over halves, base
10000, ``inv_freq = base^(-2i/d)``); the kernel (csrc/rope_embed.cu) reads q and k straight out
of the fused QKV projection output and keeps the cos/sin table in fp32.
"""
from __future__ import annotations

import torch

from . import _lib
from .gemm import LAUNCHES


def rotary_tables(rot_dim: int, max_pos: int, base: float = 10000.0, device="cpu"):
    """cos/sin tables [max_pos, rot_dim // 2] in fp32."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float32, device=device)
    freqs = torch.outer(t, inv_freq)
    return freqs.cos().contiguous(), freqs.sin().contiguous()


def _launch(x, out, cos, sin, rot, pos0, inverse):
    S, B, NH, D = x.shape
    assert x.stride(3) == 1 and out.stride(3) == 1
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(x).nx_rope(_lib.ptr(x), _lib.ptr(out), _lib.ptr(cos), _lib.ptr(sin), S, B, NH, D, rot,
                                  x.stride(0), x.stride(1), x.stride(2), out.stride(0), out.stride(1),
                                  out.stride(2), int(pos0), int(inverse), _lib.stream()), "nx_rope")


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, rot, pos0):
        out = torch.empty(x.shape, device=x.device, dtype=x.dtype)
        _launch(x, out, cos, sin, rot, pos0, False)
        ctx.save_for_backward(cos, sin)
        ctx.rot, ctx.pos0 = rot, pos0
        return out

    @staticmethod
    def backward(ctx, gy):
        cos, sin = ctx.saved_tensors
        if gy.stride(3) != 1:
            gy = gy.contiguous()
        gx = torch.empty(gy.shape, device=gy.device, dtype=gy.dtype)
        _launch(gy, gx, cos, sin, ctx.rot, ctx.pos0, True)
        return gx, None, None, None, None


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot_dim: int, pos0: int = 0):
    """x: [s, b, heads, hn] (any strides with a contiguous last dim); rotates the first ``rot_dim``
    dims of each head with positions pos0 .. pos0+s-1, passes the rest through."""
    if rot_dim == 0:
        return x
    if x.is_cuda and x.dtype in _lib.H16:
        return _RopeFn.apply(x, cos, sin, rot_dim, pos0)
    if x.is_cuda:
        raise _lib.KernelError("apply_rotary: CUDA path needs bf16")
    S = x.shape[0]
    half = rot_dim // 2
    c = cos[pos0:pos0 + S].to(x.dtype)[:, None, None, :]
    s = sin[pos0:pos0 + S].to(x.dtype)[:, None, None, :]
    x1, x2, rest = x[..., :half], x[..., half:rot_dim], x[..., rot_dim:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)
