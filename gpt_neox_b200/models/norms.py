"""Normalisation layers and their selector (megatron/model/norms.py:19-117,
megatron/model/fused_layer_norm.py). Every variant runs on this library's norm kernels for CUDA
bf16 inputs; the ``*_fusion`` switches of the reference are accepted and select nothing
different, since the fused kernel is the only CUDA implementation here."""
from __future__ import annotations

import numbers

import torch
import torch.nn as nn

from ..ops import norm as norm_ops


class LayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, no_persist_layer_norm=True, mem_efficient_ln=True):
        super().__init__()
        if isinstance(normalized_shape, numbers.Integral):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(self.normalized_shape))
        self.bias = nn.Parameter(torch.zeros(self.normalized_shape))

    def forward(self, x, carry=False):
        """``carry``: return ``(x, y)`` with the residual stream routed through the norm's autograd node
        (its gradient is then added inside the norm's backward kernel)."""
        n = len(self.normalized_shape)
        if n == 1:
            return norm_ops.layer_norm(x, self.weight, self.bias, self.eps, carry=carry)
        assert not carry
        # multi-dim normalised shape (e.g. QK-norm over [heads, head_dim]): flatten the tail
        shp = x.shape
        flat = x.reshape(*shp[:-n], -1)
        return norm_ops.layer_norm(flat, self.weight.reshape(-1), self.bias.reshape(-1), self.eps).view(shp)


class NonParametricLayernorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, x):
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), None, None, self.eps)


class RMSNorm(nn.Module):
    """x * rsqrt(mean(x^2) + eps) * scale, statistics in fp32; ``p`` in [0, 1] normalises only the
    first ``int(dim * p)`` features (partial RMSNorm), ``bias`` adds an offset."""

    def __init__(self, dim, p=-1.0, eps=1e-8, bias=False):
        super().__init__()
        if not isinstance(dim, numbers.Integral):
            d = 1
            for v in dim:
                d *= v
            self.shape_tail = tuple(dim)
            dim = d
        else:
            self.shape_tail = (dim,)
        self.eps, self.d, self.p, self.use_bias = eps, dim, p, bias
        self.scale = nn.Parameter(torch.ones(dim))
        if bias:
            self.offset = nn.Parameter(torch.zeros(dim))

    def forward(self, x, carry=False):
        if carry:
            if len(self.shape_tail) == 1 and not (0.0 <= self.p <= 1.0) and not self.use_bias:
                return norm_ops.rms_norm(x, self.scale, self.eps, carry=True)
            return x, self.forward(x)
        n = len(self.shape_tail)
        shp = x.shape
        if n > 1:
            x = x.reshape(*shp[:-n], -1)
        if 0.0 <= self.p <= 1.0:
            part = int(self.d * self.p)
            xf = x[..., :part].float()
            var = xf.pow(2).mean(-1, keepdim=True)
            out = (self.scale.float() * (x.float() * torch.rsqrt(var + self.eps)))
            out = out + self.offset.float() if self.use_bias else out
            return out.to(x.dtype).view(shp)
        out = norm_ops.rms_norm(x, self.scale, self.eps)
        if self.use_bias:
            out = out + self.offset
        return out.view(shp)


class ScaleNorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.g = nn.Parameter(torch.ones(1))
        self.eps = eps

    def forward(self, x):
        n = torch.norm(x, dim=-1, keepdim=True).clamp(min=self.eps)
        return x / n * self.g


def get_norm(neox_args):
    """-> (norm class, eps). ``te_rmsnorm`` / ``te_layernorm`` map onto the same kernels."""
    name = neox_args.norm
    if name in ("rmsnorm", "te_rmsnorm"):
        return RMSNorm, neox_args.rms_norm_epsilon
    if name in ("layernorm", "te_layernorm"):
        return LayerNorm, neox_args.layernorm_epsilon
    if name == "non_parametric_layernorm":
        if neox_args.layernorm_fusion:
            raise ValueError("neox_args.layernorm_fusion not supported for non_parametric_layernorm")
        return NonParametricLayernorm, neox_args.layernorm_epsilon
    if name == "scalenorm":
        return ScaleNorm, neox_args.scalenorm_epsilon
    raise ValueError(f"norm {name} not recognized")
