"""Activations (plain and gated), bias+dropout+residual, column sums.

CUDA bf16 tensors run csrc/elementwise.cu; CPU tensors run the PyTorch statement of the same math
(megatron/model/activations.py:27-135, megatron/model/transformer.py:182-198,
megatron/model/fused_bias_dropout.py:28-55).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import LAUNCHES

ACT_IDS = {"gelu": 0, "gelu_tanh": 1, "relu": 2, "silu": 3, "swish": 3, "identity": 4,
           "sigmoid": 5, "relu2": 6}
#: gated activation name -> activation applied to the gate half
GATED = {"geglu": "gelu", "reglu": "relu", "bilinear": "identity", "swiglu": "silu", "glu": "sigmoid"}


def _torch_act(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "gelu":
        return F.gelu(x)
    if name == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    if name == "relu":
        return F.relu(x)
    if name in ("silu", "swish"):
        return F.silu(x)
    if name == "identity":
        return x
    if name == "sigmoid":
        return torch.sigmoid(x)
    if name == "relu2":
        return F.relu(x) ** 2
    if name == "softsign":
        return F.softsign(x)
    if name == "mish":
        return x * torch.tanh(F.softplus(x))
    raise ValueError(f"activation {name} not recognized")


def _cuda_ok(x):
    return x.is_cuda and x.dtype in _lib.H16 and x.shape[-1] % 8 == 0


def colsum(x2: torch.Tensor, out_dtype=None, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Sum over rows of a 2-D bf16 tensor (bias gradient); fp32 accumulation.  ``out`` (fp32 or the input's dtype, N
    contiguous elements) receives the sums, added to its contents with ``accumulate``."""
    if not x2.is_cuda:
        r = x2.float().sum(0)
        if out is not None:
            out.copy_(out.float() + r if accumulate else r)
            return out
        return r.to(out_dtype or x2.dtype)
    rows, N = x2.shape
    L = _lib.lib(x2)
    slabs = L.nx_colsum_slabs(rows)
    ws = torch.empty(slabs * N, device=x2.device, dtype=torch.float32)
    out_dtype = out.dtype if out is not None else (out_dtype or x2.dtype)
    if out is None:
        out = torch.empty(N, device=x2.device, dtype=out_dtype)
    LAUNCHES["n"] += 2
    _lib.check(L.nx_colsum_bf16(
        _lib.ptr(x2), _lib.ptr(out) if out_dtype == torch.float32 else None,
        _lib.ptr(out) if out_dtype == x2.dtype else None, _lib.ptr(ws), rows, N, x2.stride(0),
        1 if accumulate else 0, _lib.stream()), "nx_colsum_bf16")
    return out


def bias_grad(x2: torch.Tensor, bias) -> torch.Tensor | None:
    """Gradient of a bias that was added to every row: the column sum of ``x2``.  When the engine gave the bias a
    fp32 ``main_grad`` the sum is added straight into it by the reduction kernel (returns None: nothing is left for
    autograd to accumulate, convert and fold in later)."""
    mg = getattr(bias, "main_grad", None)
    if (mg is not None and x2.is_cuda and mg.dtype == torch.float32 and mg.is_contiguous()
            and mg.numel() == x2.shape[1]):
        colsum(x2, out=mg.view(-1), accumulate=True)
        return None
    return colsum(x2)


class _BiasActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, act_id):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = torch.empty_like(x2)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x2).nx_bias_act_fwd(_lib.ptr(x2), _lib.ptr(bias), _lib.ptr(y), x2.shape[0],
                                              x2.shape[1], act_id, _lib.stream()), "nx_bias_act_fwd")
        ctx.save_for_backward(x2, bias)
        ctx.act_id, ctx.shape = act_id, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        x2, bias = ctx.saved_tensors
        gy2 = gy.reshape(x2.shape).contiguous()
        dx = torch.empty_like(x2)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(gy2).nx_bias_act_bwd(_lib.ptr(gy2), _lib.ptr(x2), _lib.ptr(bias), _lib.ptr(dx),
                                              x2.shape[0], x2.shape[1], ctx.act_id, _lib.stream()),
                   "nx_bias_act_bwd")
        gb = colsum(dx) if (bias is not None and ctx.needs_input_grad[1]) else None
        return dx.view(ctx.shape), gb, None


def bias_act(x: torch.Tensor, bias: torch.Tensor | None, act: str) -> torch.Tensor:
    """``act(x + bias)``; act in ACT_IDS (CUDA) or any name ``_torch_act`` knows (CPU)."""
    if _cuda_ok(x) and act in ACT_IDS:
        return _BiasActFn.apply(x, bias, ACT_IDS[act])
    if x.is_cuda and act in ACT_IDS:
        raise _lib.KernelError("bias_act: CUDA path needs bf16 and last dim % 8 == 0")
    return _torch_act(act, x if bias is None else x + bias)


class _GatedActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, act_id):
        F2 = x.shape[-1]
        x2 = x.reshape(-1, F2).contiguous()
        y = torch.empty((x2.shape[0], F2 // 2), device=x.device, dtype=x.dtype)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x2).nx_gated_act_fwd(_lib.ptr(x2), _lib.ptr(y), x2.shape[0], F2 // 2, act_id,
                                               _lib.stream()), "nx_gated_act_fwd")
        ctx.save_for_backward(x2)
        ctx.act_id, ctx.shape = act_id, x.shape
        return y.view(*x.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, gy):
        (x2,) = ctx.saved_tensors
        gy2 = gy.reshape(x2.shape[0], -1).contiguous()
        dx = torch.empty_like(x2)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(gy2).nx_gated_act_bwd(_lib.ptr(gy2), _lib.ptr(x2), _lib.ptr(dx), x2.shape[0],
                                               x2.shape[1] // 2, ctx.act_id, _lib.stream()),
                   "nx_gated_act_bwd")
        return dx.view(ctx.shape), None


def gated_act(x: torch.Tensor, kind: str) -> torch.Tensor:
    """x = [value | gate] along the last dim; returns ``value * act(gate)``
    (chunk order of megatron/model/transformer.py:189-198)."""
    act = GATED[kind]
    if _cuda_ok(x) and (x.shape[-1] // 2) % 8 == 0:
        return _GatedActFn.apply(x, ACT_IDS[act])
    if x.is_cuda:
        raise _lib.KernelError("gated_act: CUDA path needs bf16 and F % 8 == 0")
    v, g = x.chunk(2, dim=-1)
    return v * _torch_act(act, g)


class _BiasDropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p, seed, offset):
        H = x.shape[-1]
        x2 = x.reshape(-1, H).contiguous()
        r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
        out = torch.empty_like(x2)
        mask = torch.empty(x2.numel() // 8, device=x.device, dtype=torch.uint8) if p > 0 else None
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x2).nx_bias_dropout_add(
            _lib.ptr(x2), _lib.ptr(bias), _lib.ptr(r2), _lib.ptr(out), _lib.ptr(mask), x2.shape[0], H,
            float(p), int(seed), int(offset), _lib.stream()), "nx_bias_dropout_add")
        ctx.p, ctx.shape, ctx.has_bias, ctx.has_res = p, x.shape, bias is not None, residual is not None
        ctx.save_for_backward(mask)
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        (mask,) = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        if ctx.p > 0:
            dx = torch.empty_like(gy2)
            LAUNCHES["n"] += 1
            _lib.check(_lib.lib(gy2).nx_dropout_bwd(_lib.ptr(gy2), _lib.ptr(mask), _lib.ptr(dx), gy2.numel(),
                                                 float(ctx.p), _lib.stream()), "nx_dropout_bwd")
        else:
            dx = gy2
        gb = colsum(dx) if ctx.has_bias else None
        return dx.view(ctx.shape), gb, (gy if ctx.has_res else None), None, None, None


_DROPOUT_OFFSET = {"n": 0}


def bias_dropout_add(x, bias, residual, p: float, training: bool):
    """``residual + dropout(x + bias, p)``; bias / residual optional."""
    p = p if training else 0.0
    if _cuda_ok(x):
        if p == 0.0 and bias is None and residual is None:
            return x
        seed = torch.initial_seed() & 0x7FFFFFFFFFFFFFFF
        _DROPOUT_OFFSET["n"] += 1
        return _BiasDropoutAddFn.apply(x, bias, residual, p, seed, _DROPOUT_OFFSET["n"])
    if x.is_cuda:
        raise _lib.KernelError("bias_dropout_add: CUDA path needs bf16 and last dim % 8 == 0")
    out = x if bias is None else x + bias
    out = F.dropout(out, p=p, training=training)
    return out if residual is None else residual + out
