"""Causal flash attention (GQA, ALiBi, sliding window) on the tcgen05 kernels of
csrc/attention_fwd.cu / csrc/attention_bwd.cu, with a PyTorch reference used on CPU and as the
test oracle.

Tensors are passed as ``[b, s, heads, hd]`` views with arbitrary batch / sequence / head strides
(the head dim contiguous), so the q / k / v slices of the fused QKV projection output are consumed
in place.  Counterpart of megatron/model/transformer.py:573-690.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from .gemm import LAUNCHES


def alibi_slopes(n_heads: int) -> torch.Tensor:
    """Per-head ALiBi slopes (megatron/model/positional_embeddings.py:146-167)."""
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(n_heads).is_integer():
        s = pow2(n_heads)
    else:
        c = 2 ** math.floor(math.log2(n_heads))
        s = pow2(c) + pow2(2 * c)[0::2][: n_heads - c]
    return torch.tensor(s, dtype=torch.float32)


def attention_reference(q, k, v, *, scale=None, causal=True, window: int = -1, alibi=None):
    """Plain PyTorch attention in fp32. q [b,sq,h,d], k/v [b,sk,hk,d] -> ([b,sq,h,d], lse [b,h,sq])."""
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qf, kf, vf = q.float(), k.float(), v.float()
    if hk != h:
        kf = kf.repeat_interleave(h // hk, dim=2)
        vf = vf.repeat_interleave(h // hk, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    qpos = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
    kpos = torch.arange(sk, device=q.device)[None, :]
    if alibi is not None:
        s = s + alibi.to(s.device).float()[None, :, None, None] * (kpos - qpos).float()[None, None]
    dead = torch.zeros(sq, sk, dtype=torch.bool, device=q.device)
    if causal:
        dead |= kpos > qpos
    if window is not None and window >= 0:
        dead |= kpos < qpos - window
    s = s.masked_fill(dead[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum("bhqk,bkhd->bqhd", p, vf)
    return o.to(q.dtype), lse


def _strides_bhs(t):
    # tensor is [b, s, h, d] -> (batch, head, seq) element strides
    return t.stride(0), t.stride(2), t.stride(1)


def _fwd(q, k, v, scale, causal, window, alibi):
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    o = torch.empty((b, sq, h, d), device=q.device, dtype=q.dtype)
    # base-2 log-sum-exp, rows padded to a multiple of 128 with +inf (the backward reads whole
    # 128-row blocks of it; +inf makes the padding contribute zero probability)
    sq_pad = (sq + 127) // 128 * 128
    lse = torch.full((b, h, sq_pad), float("inf"), device=q.device, dtype=torch.float32)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(q).nx_flash_attn_fwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(alibi),
        b, h, hk, sq, sk, d, *_strides_bhs(q), *_strides_bhs(k), *_strides_bhs(v), *_strides_bhs(o),
        float(scale), int(causal), int(window), _lib.stream()), "nx_flash_attn_fwd")
    return o, lse


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, window, alibi):
        o, lse = _fwd(q, k, v, scale, causal, window, alibi)
        ctx.save_for_backward(q, k, v, o, lse, alibi)
        ctx.scale, ctx.causal, ctx.window = scale, causal, window
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, alibi = ctx.saved_tensors
        b, sq, h, d = q.shape
        sk, hk = k.shape[1], k.shape[2]
        if do.stride(3) != 1 or any(s % 8 for s in do.stride()[:3]):
            do = do.contiguous()
        dq = torch.empty((b, sq, h, d), device=q.device, dtype=q.dtype)
        dk = torch.empty((b, sk, hk, d), device=q.device, dtype=q.dtype)
        dv = torch.empty((b, sk, hk, d), device=q.device, dtype=q.dtype)
        delta = torch.zeros(lse.shape, device=q.device, dtype=torch.float32)
        LAUNCHES["n"] += 3
        _lib.check(_lib.lib(q).nx_flash_attn_bwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse),
            _lib.ptr(delta), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(alibi),
            b, h, hk, sq, sk, d, *_strides_bhs(q), *_strides_bhs(k), *_strides_bhs(v), *_strides_bhs(o),
            *_strides_bhs(do), *_strides_bhs(dq), *_strides_bhs(dk), *_strides_bhs(dv),
            float(ctx.scale), int(ctx.causal), int(ctx.window), _lib.stream()), "nx_flash_attn_bwd")
        return dq, dk, dv, None, None, None, None


def flash_attention(q, k, v, *, scale: float | None = None, causal: bool = True, window: int = -1,
                    alibi: torch.Tensor | None = None) -> torch.Tensor:
    """q [b,sq,h,d]; k, v [b,sk,hk,d] (h % hk == 0). Query i sits at position i + (sk - sq)."""
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    window = -1 if window is None else int(window)
    if q.is_cuda:
        if q.dtype not in _lib.H16 or d % 8 or d > 128:
            raise _lib.KernelError(f"flash_attention: CUDA path needs bf16 and head dim % 8 == 0, <= 128 (got {q.dtype}, {d})")
        fix = lambda t: t if (t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0) else t.contiguous()
        if alibi is not None:
            alibi = alibi.to(device=q.device, dtype=torch.float32).contiguous()
        return _FlashAttnFn.apply(fix(q), fix(k), fix(v), scale, causal, window, alibi)
    return attention_reference(q, k, v, scale=scale, causal=causal, window=window, alibi=alibi)[0]
