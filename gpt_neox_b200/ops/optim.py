"""Flat fused AdamW, sum-of-squares and clip coefficient (csrc/optim.cu); PyTorch on CPU."""
from __future__ import annotations

import torch

from . import _lib
from .gemm import LAUNCHES


def sumsq_(x: torch.Tensor, acc: torch.Tensor):
    """acc[0] += sum(x^2); acc[1] = 1 if a non-finite value was seen. acc: float32[2]."""
    if x.numel() == 0:
        return
    if x.is_cuda:
        assert x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float16, torch.float32)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x).nx_sumsq(_lib.ptr(x), x.numel(), _lib.ptr(acc), 1 if x.dtype == torch.float32 else 0,
                                       _lib.stream()), "nx_sumsq")
    else:
        s = x.float().pow(2).sum()
        acc[0] += s
        if not torch.isfinite(s):
            acc[1] = 1.0


def clip_coef_(acc: torch.Tensor, max_norm: float, inv_scale: float, out: torch.Tensor, skip: torch.Tensor):
    """out[0] = gradient multiplier (clip coefficient x inv_scale), out[1] = global norm,
    skip[0] = 1 if gradients were non-finite. All on device, no host sync."""
    if acc.is_cuda:
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib().nx_clip_coef(_lib.ptr(acc), float(max_norm), float(inv_scale), _lib.ptr(out),
                                           _lib.ptr(skip), _lib.stream()), "nx_clip_coef")
    else:
        norm = acc[0].sqrt() * inv_scale
        coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.tensor(1.0)
        out[0] = coef * inv_scale
        out[1] = norm
        skip[0] = int(bool(acc[1] != 0) or not bool(torch.isfinite(norm)))


def adamw_step_(p32, m, v, g, p_lp, *, lr, beta1, beta2, eps, weight_decay, step, adam_w_mode=True,
                grad_scale=None, skip=None):
    """One AdamW update of a flat fp32 shard; writes the low-precision copy ``p_lp`` if given.
    ``grad_scale``: device float tensor multiplying the gradient; ``skip``: device int, non-zero = no-op."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if p32.is_cuda:
        assert p32.is_contiguous() and g.is_contiguous()
        LAUNCHES["n"] += 1
        lp16 = p_lp is not None and p_lp.dtype in _lib.H16
        assert g.dtype == torch.float32 or not lp16 or g.dtype == p_lp.dtype, (g.dtype, p_lp.dtype)
        _lib.check(_lib.lib(p_lp if lp16 else g).nx_adamw_step(
            _lib.ptr(p32), _lib.ptr(m), _lib.ptr(v), _lib.ptr(g),
            _lib.ptr(p_lp) if lp16 else None,
            p32.numel(), float(lr), float(beta1), float(beta2), float(eps), float(weight_decay),
            float(bc1), float(bc2), int(adam_w_mode), _lib.ptr(grad_scale), _lib.ptr(skip),
            1 if g.dtype == torch.float32 else 0, _lib.stream()), "nx_adamw_step")
        if p_lp is not None and not lp16:
            p_lp.copy_(p32)
        return
    if skip is not None and int(skip[0]) != 0:
        return
    gf = g.float()
    if grad_scale is not None:
        gf = gf * grad_scale[0]
    if not adam_w_mode:
        gf = gf + weight_decay * p32
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    denom = v.sqrt() / (bc2 ** 0.5) + eps
    if adam_w_mode:
        p32.mul_(1 - lr * weight_decay)
    p32.addcdiv_(m, denom, value=-lr / bc1)
    if p_lp is not None:
        p_lp.copy_(p32)
