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
    return x.is_cuda and x.dtype in _lib.H16 and x.shape[-1] % 8 == 0


def _accum_param_grad(param: torch.Tensor, g_f32: torch.Tensor):
    """Route a fp32 parameter gradient: into ``main_grad`` if the engine installed one."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        mg.add_(g_f32.view_as(mg))
        return None
    return g_f32.to(param.dtype)


class _NormFn(torch.autograd.Function):
    """One or two norms of ``x``.  ``carry``: also return ``x`` itself as the first output, so that the
    gradient of the residual stream flows through this node and is added inside the backward kernel
    (no separate accumulation pass over the activations)."""

    @staticmethod
    def forward(ctx, kind, x, gamma, beta, eps, gamma2, beta2, carry):
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
        _lib.check(_lib.lib(x2).nx_norm_fwd(
            kind, _lib.ptr(x2), _lib.ptr(gamma), _lib.ptr(beta), _lib.ptr(y1), _lib.ptr(gamma2),
            _lib.ptr(beta2), _lib.ptr(y2), _lib.ptr(mean), _lib.ptr(rstd), rows, H, float(eps),
            _lib.stream()), "nx_norm_fwd")
        ctx.kind, ctx.dual, ctx.shape, ctx.carry = kind, dual, x.shape, carry
        ctx.has_beta = beta is not None
        ctx.has_beta2 = beta2 is not None
        ctx.params = tuple(getattr(t, "_nx_param", None) for t in (gamma, beta, gamma2, beta2))
        ctx.save_for_backward(x2, gamma, gamma2, mean, rstd)
        outs = (y1.view(x.shape),) + ((y2.view(x.shape),) if dual else ())
        if carry:
            return (x2.view(x.shape),) + outs
        return outs if dual else outs[0]

    @staticmethod
    def backward(ctx, *gys):
        x2, gamma, gamma2, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        L = _lib.lib(x2)

        def flat(t):
            if t is None:
                return None
            t = t.reshape(rows, H)
            return t if t.is_contiguous() else t.contiguous()

        gres = flat(gys[0]) if ctx.carry else None
        gys = gys[1:] if ctx.carry else gys
        g1 = flat(gys[0])
        g2 = flat(gys[1]) if ctx.dual else None
        pairs = [(g, gm, hb) for g, gm, hb in ((g1, gamma, ctx.has_beta), (g2, gamma2, ctx.has_beta2))
                 if g is not None]
        new = lambda: torch.empty(H, device=x2.device, dtype=torch.float32)
        grads = {}
        dx = gres
        if pairs:
            (ga, gma, hba), (gb, gmb, hbb) = pairs[0], (pairs[1] if len(pairs) == 2 else (None, None, False))
            blocks = L.nx_norm_bwd_blocks(rows)
            ws = torch.empty(blocks * (4 if gb is not None else 2) * H, device=x2.device, dtype=torch.float32)
            dx = torch.empty_like(x2)
            # parameter gradients: straight into the fp32 main_grad buffers (added by the partial-sum reduction
            # kernel) when every parameter of this call has one, else into fresh buffers that autograd routes
            owners = {id(gamma): ctx.params[0:2], id(gamma2): ctx.params[2:4]} if ctx.dual else {id(gamma): ctx.params[0:2]}
            want = [owners[id(gma)][0]] + ([owners[id(gma)][1]] if hba else [])
            if gb is not None:
                want += [owners[id(gmb)][0]] + ([owners[id(gmb)][1]] if hbb else [])
            mgs = [getattr(p_, "main_grad", None) if p_ is not None else None for p_ in want]
            direct = all(m is not None and m.dtype == torch.float32 and m.is_contiguous() and m.numel() == H for m in mgs)
            if direct:
                it = iter(mgs)
                dga, dba = next(it), (next(it) if hba else None)
                dgb, dbb = (next(it) if gb is not None else None), (next(it) if (gb is not None and hbb) else None)
            else:
                dga, dba = new(), (new() if hba else None)
                dgb, dbb = (new() if gb is not None else None), (new() if hbb else None)
            LAUNCHES["n"] += 2
            _lib.check(L.nx_norm_bwd(
                ctx.kind, _lib.ptr(ga), _lib.ptr(gb), _lib.ptr(x2), _lib.ptr(mean), _lib.ptr(rstd),
                _lib.ptr(gma), _lib.ptr(gmb), _lib.ptr(gres), _lib.ptr(dx), _lib.ptr(dga), _lib.ptr(dba),
                _lib.ptr(dgb), _lib.ptr(dbb), _lib.ptr(ws), rows, H, 1 if direct else 0, _lib.stream()), "nx_norm_bwd")
            if not direct:
                grads[id(gma)] = (dga, dba)
                if gb is not None:
                    grads[id(gmb)] = (dgb, dbb)
        d1 = grads.get(id(gamma), (None, None))
        d2 = grads.get(id(gamma2), (None, None)) if ctx.dual else (None, None)
        return (None, dx.view(ctx.shape) if dx is not None else None, d1[0], d1[1], None, d2[0], d2[1], None)


class _ParamGrad(torch.autograd.Function):
    """Identity on a parameter whose backward converts the fp32 kernel gradient to the
    parameter's dtype (or accumulates it into ``param.main_grad``)."""

    @staticmethod
    def forward(ctx, p):
        ctx.p = p
        ctx.set_materialize_grads(False)      # no gradient arrives when the norm kernel wrote into main_grad itself
        return p.detach()

    @staticmethod
    def backward(ctx, g):
        return None if g is None else _accum_param_grad(ctx.p, g)


def _wrap(p):
    if p is None or not p.requires_grad:
        return p
    w = _ParamGrad.apply(p)
    w._nx_param = p          # the norm's backward adds into p.main_grad itself when it can (see _NormFn.backward)
    return w


def layer_norm(x, weight, bias=None, eps: float = 1e-5, carry: bool = False):
    """``carry``: return ``(x, y)``; the gradient of that ``x`` (the residual stream) is added to the
    norm's input gradient inside the backward kernel."""
    if _cuda_ok(x):
        return _NormFn.apply(LN, x, _wrap(weight), _wrap(bias), eps, None, None, carry)
    if carry:
        return x, layer_norm(x, weight, bias, eps)
    if x.is_cuda:
        raise _lib.KernelError(f"layer_norm: CUDA path needs bf16 and H % 8 == 0, got {x.dtype} {tuple(x.shape)}")
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def dual_layer_norm(x, w1, b1, w2, b2, eps: float = 1e-5, carry: bool = False):
    """Two LayerNorms of the same input from one pass (GPT-J parallel residual,
    megatron/model/transformer.py:1083).  ``carry``: return ``(x, y1, y2)`` where the first output
    stands for the residual stream; its gradient is added to the norms' input gradient inside the
    backward kernel."""
    if _cuda_ok(x):
        return _NormFn.apply(LN, x, _wrap(w1), _wrap(b1), eps, _wrap(w2), _wrap(b2), carry)
    y = layer_norm(x, w1, b1, eps), layer_norm(x, w2, b2, eps)
    return (x,) + y if carry else y


def rms_norm(x, weight, eps: float = 1e-8, carry: bool = False):
    if _cuda_ok(x):
        return _NormFn.apply(RMS, x, _wrap(weight), None, eps, None, None, carry)
    if carry:
        return x, rms_norm(x, weight, eps)
    if x.is_cuda:
        raise _lib.KernelError(f"rms_norm: CUDA path needs bf16 and H % 8 == 0, got {x.dtype}")
    dtype = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (weight.float() * (xf * torch.rsqrt(var + eps))).to(dtype)


def dual_rms_norm(x, w1, w2, eps: float = 1e-8):
    if _cuda_ok(x):
        return _NormFn.apply(RMS, x, _wrap(w1), None, eps, _wrap(w2), None, False)
    return rms_norm(x, w1, eps), rms_norm(x, w2, eps)
