"""Flat fused AdamW, sum-of-squares and clip coefficient (csrc/optim.cu); PyTorch on CPU."""
from __future__ import annotations

import math

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


# ---------------------------------------------------------------------------------------------------------------
# AdamW with 8-bit block-wise state (``use_bnb_optimizer``; csrc/optim.cu adam8_kernel).  The PyTorch functions
# below state the same code (one byte per moment element, one fp32 scale per 2048 elements) and are the CPU path.
# ---------------------------------------------------------------------------------------------------------------
Q8_BLOCK = 2048
_Q8_M_STEP, _Q8_V_STEP = 14.0 / 126.0, 28.0 / 254.0


def q8_blocks(n: int) -> int:
    return (n + Q8_BLOCK - 1) // Q8_BLOCK


def _per_element(scale, n):
    return scale.repeat_interleave(Q8_BLOCK)[:n]


def q8_decode(m8, v8, scale_m, scale_v):
    """uint8 codes + block scales -> fp32 moments."""
    n = m8.numel()
    b = m8.to(torch.int32)
    c = (b & 127).float()
    mag = torch.where(c == 0, torch.zeros_like(c), _per_element(scale_m, n) * torch.exp2((c - 127.0) * _Q8_M_STEP))
    m = torch.where((b & 128) != 0, -mag, mag)
    cv = v8.float()
    v = torch.where(cv == 0, torch.zeros_like(cv), _per_element(scale_v, n) * torch.exp2((cv - 255.0) * _Q8_V_STEP))
    return m, v


def q8_encode(m, v):
    """fp32 moments -> (m8, v8, scale_m, scale_v)."""
    n = m.numel()
    pad = q8_blocks(n) * Q8_BLOCK - n
    mp = torch.nn.functional.pad(m.abs(), (0, pad)).view(-1, Q8_BLOCK)
    vp = torch.nn.functional.pad(v, (0, pad)).view(-1, Q8_BLOCK)
    scale_m, scale_v = mp.max(dim=1).values, vp.max(dim=1).values
    sm, sv = _per_element(scale_m, n), _per_element(scale_v, n)
    rm = torch.where(sm > 0, m.abs() / sm.clamp_min(1e-45), torch.zeros_like(m))
    rv = torch.where(sv > 0, v / sv.clamp_min(1e-45), torch.zeros_like(v))
    cm = torch.where(rm > 0, torch.round(127.0 + torch.log2(rm.clamp_min(1e-45)) / _Q8_M_STEP), torch.zeros_like(rm))
    cv = torch.where(rv > 0, torch.round(255.0 + torch.log2(rv.clamp_min(1e-45)) / _Q8_V_STEP), torch.zeros_like(rv))
    m8 = cm.clamp(0, 127).to(torch.int32) | torch.where(m < 0, 128, 0).to(torch.int32)
    return m8.to(torch.uint8), cv.clamp(0, 255).to(torch.uint8), scale_m, scale_v


def adamw8bit_step_(p32, m8, v8, scale_m, scale_v, g, p_lp, *, lr, beta1, beta2, eps, weight_decay, step,
                    adam_w_mode=True, grad_scale=None, skip=None):
    """One AdamW update of a flat fp32 shard whose moments are stored in 8 bits (in place on every argument)."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    n = p32.numel()
    assert scale_m.numel() == q8_blocks(n) and scale_v.numel() == q8_blocks(n)
    if p32.is_cuda:
        assert n % 8 == 0 and p32.is_contiguous() and g.is_contiguous()
        lp16 = p_lp is not None and p_lp.dtype in _lib.H16
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(p_lp if lp16 else g).nx_adamw8bit_step(
            _lib.ptr(p32), _lib.ptr(m8), _lib.ptr(v8), _lib.ptr(scale_m), _lib.ptr(scale_v), _lib.ptr(g),
            _lib.ptr(p_lp) if lp16 else None, n, float(lr), float(beta1), float(beta2), float(eps),
            float(weight_decay), float(bc1), float(bc2), int(adam_w_mode), _lib.ptr(grad_scale), _lib.ptr(skip),
            1 if g.dtype == torch.float32 else 0, _lib.stream()), "nx_adamw8bit_step")
        if p_lp is not None and not lp16:
            p_lp.copy_(p32)
        return
    if skip is not None and int(skip[0]) != 0:
        return
    m, v = q8_decode(m8, v8, scale_m, scale_v)
    gs = float(grad_scale[0]) if grad_scale is not None else 1.0
    gr = g.float() * gs
    if not adam_w_mode:
        gr = gr + weight_decay * p32
    m = beta1 * m + (1 - beta1) * gr
    v = beta2 * v + (1 - beta2) * gr * gr
    if adam_w_mode:
        p32.mul_(1 - lr * weight_decay)
    p32.addcdiv_(m, v.sqrt() / math.sqrt(bc2) + eps, value=-lr / bc1)
    a, b, c, d = q8_encode(m, v)
    m8.copy_(a), v8.copy_(b), scale_m.copy_(c), scale_v.copy_(d)
    if p_lp is not None:
        p_lp.copy_(p32)


# ---------------------------------------------------------------------------------------------------------------
# Host AdamW for optimizer-state offload (csrc/cpu_adam.cpp -> lib/libneox_host.so)
# ---------------------------------------------------------------------------------------------------------------
_HOST_LIB = [None]


def _host_lib():
    if _HOST_LIB[0] is None:
        import ctypes as C
        from pathlib import Path
        path = Path(__file__).resolve().parent.parent / "lib" / "libneox_host.so"
        if not path.exists():
            from ..build import build_host_ops
            build_host_ops()
        L = C.CDLL(str(path))
        F, I, P = C.c_float, C.c_int, C.c_void_p
        L.nx_cpu_adamw.argtypes = [P, P, P, P, I, P, I, C.c_longlong, F, F, F, F, F, F, F, I, F, I]
        L.nx_cpu_adamw.restype = I
        _HOST_LIB[0] = L
    return _HOST_LIB[0]


_KIND = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}


def cpu_adamw_step_(p32, m, v, g, p_lp, *, lr, beta1, beta2, eps, weight_decay, step, adam_w_mode=True,
                    grad_scale: float = 1.0, threads: int = 0):
    """AdamW on host tensors with the native multi-threaded kernel: ``p32`` / ``m`` / ``v`` fp32, ``g`` bf16 / fp16 /
    fp32, ``p_lp`` (optional) receives the new weights as bf16 / fp16.  All contiguous CPU tensors, updated in place."""
    import ctypes as C
    for t in (p32, m, v, g) + ((p_lp,) if p_lp is not None else ()):
        assert t.device.type == "cpu" and t.is_contiguous()
    assert p32.dtype == m.dtype == v.dtype == torch.float32 and g.dtype in _KIND and g.numel() == p32.numel()
    lp16 = p_lp is not None and p_lp.dtype in (torch.bfloat16, torch.float16)
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    _host_lib().nx_cpu_adamw(C.c_void_p(p32.data_ptr()), C.c_void_p(m.data_ptr()), C.c_void_p(v.data_ptr()),
                             C.c_void_p(g.data_ptr()), _KIND[g.dtype], C.c_void_p(p_lp.data_ptr()) if lp16 else None,
                             _KIND[p_lp.dtype] if lp16 else 0, p32.numel(), float(lr), float(beta1), float(beta2),
                             float(eps), float(weight_decay), float(bc1), float(bc2), int(adam_w_mode),
                             float(grad_scale), int(threads))
    if p_lp is not None and not lp16:
        p_lp.copy_(p32)
