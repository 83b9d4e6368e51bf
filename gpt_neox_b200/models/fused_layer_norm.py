"""``MixedFusedLayerNorm`` / ``MixedFusedRMSNorm`` with the reference's constructor arguments
(megatron/model/fused_layer_norm.py:34-229), on this library's norm kernels.

``apply_layernorm_1p`` / ``apply_rmsnorm_1p`` store the scale as ``weight - 1`` (zero-initialised, so weight
decay pulls the effective scale towards one).  ``no_persist_layer_norm`` and ``mem_efficient_*`` select
between apex kernels in the reference; here there is one kernel per norm, which keeps only the row statistics
for backward, so the flags are accepted and change nothing.  ``sequence_parallel`` marks the parameters so the
engine sums their gradients over the tensor-parallel group.
"""
from __future__ import annotations

import numbers

import torch
import torch.nn as nn

from ..ops import norm as norm_ops


def _shape(normalized_shape):
    if isinstance(normalized_shape, numbers.Integral):
        return (int(normalized_shape),)
    return tuple(int(v) for v in normalized_shape)


class MixedFusedLayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, no_persist_layer_norm=True, sequence_parallel=False,
                 apply_layernorm_1p=False, mem_efficient_ln=True):
        super().__init__()
        self.normalized_shape = _shape(normalized_shape)
        self.eps, self.apply_layernorm_1p = eps, apply_layernorm_1p
        self.no_persist_layer_norm, self.mem_efficient_ln = no_persist_layer_norm, mem_efficient_ln
        self.sequence_parallel = sequence_parallel
        self.weight = nn.Parameter(torch.empty(self.normalized_shape))
        self.bias = nn.Parameter(torch.empty(self.normalized_shape))
        self.reset_parameters()
        for p in (self.weight, self.bias):
            p.sequence_parallel = sequence_parallel
            if sequence_parallel:
                p.sequence_parallel_grad_sync = True

    def reset_parameters(self):
        nn.init.zeros_(self.weight) if self.apply_layernorm_1p else nn.init.ones_(self.weight)
        nn.init.zeros_(self.bias)

    def forward(self, input):
        w = self.weight + 1 if self.apply_layernorm_1p else self.weight
        n = len(self.normalized_shape)
        shp = input.shape
        flat = input.reshape(*shp[:-n], -1) if n > 1 else input
        return norm_ops.layer_norm(flat, w.reshape(-1), self.bias.reshape(-1), self.eps).view(shp)


class MixedFusedRMSNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, no_persist_layer_norm=True, sequence_parallel=False,
                 apply_rmsnorm_1p=False, mem_efficient_rms=True):
        super().__init__()
        self.normalized_shape = _shape(normalized_shape)
        self.eps, self.apply_rmsnorm_1p = eps, apply_rmsnorm_1p
        self.no_persist_layer_norm, self.mem_efficient_rms = no_persist_layer_norm, mem_efficient_rms
        self.sequence_parallel = sequence_parallel
        self.scale = nn.Parameter(torch.empty(self.normalized_shape))
        self.reset_parameters()
        self.scale.sequence_parallel = sequence_parallel
        if sequence_parallel:
            self.scale.sequence_parallel_grad_sync = True

    def reset_parameters(self):
        nn.init.zeros_(self.scale) if self.apply_rmsnorm_1p else nn.init.ones_(self.scale)

    def forward(self, input):
        w = self.scale + 1 if self.apply_rmsnorm_1p else self.scale
        n = len(self.normalized_shape)
        shp = input.shape
        flat = input.reshape(*shp[:-n], -1) if n > 1 else input
        return norm_ops.rms_norm(flat, w.reshape(-1), self.eps).view(shp)
