"""The reference's Transformer-Engine adapter names (megatron/model/transformer_engine.py:58-670) on this
library's own fp8 path: no Transformer Engine is imported.

* `TEColumnParallelLinear` / `TERowParallelLinear` / `TELinear`: the parallel linears with their GEMMs on the
  fp8 tensor-core kernel (e4m3 forward operands, e5m2 or e4m3 gradients, per-tensor delayed scaling kept on the
  device);
* `TELayerNormMLP`: norm + MLP block with both GEMMs in fp8;
* `TERMSNorm` / `TELayerNorm`: the norm kernels;
* `TEMultiheadAttention`: the attention block (the bf16 flash kernel serves ``te_mha`` / ``te_fp8_mha``);
* `TEDelayedScaling`: the recipe object (format, margin, amax history length and reduction); its
  ``fp8_context()`` is a no-op context manager because fp8 is a property of the modules here, not of a scope.
"""
from __future__ import annotations

import contextlib
import copy

import torch
import torch.nn as nn

from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from .norms import LayerNorm, RMSNorm


def _with(neox_args, **flags):
    a = copy.copy(neox_args)
    for k, v in flags.items():
        setattr(a, k, v)
    return a


class TERMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-8, **kwargs):
        super().__init__()
        self.d, self.eps = dim, eps
        self.norm = RMSNorm(dim, eps=eps)

    def forward(self, x):
        return self.norm(x)


class TELayerNorm(nn.Module):
    def __init__(self, dim, eps=1.0e-5, **kwargs):
        super().__init__()
        self.d, self.eps = dim, eps
        self.norm = LayerNorm(dim, eps=eps)

    def forward(self, x):
        return self.norm(x)


class TEColumnParallelLinear(ColumnParallelLinear):
    def __init__(self, neox_args, *args, **kwargs):
        super().__init__(_with(neox_args, te_columnparallel=True), *args, **kwargs)


class TERowParallelLinear(RowParallelLinear):
    def __init__(self, neox_args, *args, **kwargs):
        super().__init__(_with(neox_args, te_rowparallel=True), *args, **kwargs)


class TELinear(TEColumnParallelLinear):
    """A linear whose output is gathered: the unsharded layer as far as the caller can tell."""

    def __init__(self, neox_args, input_size, output_size, bias=True, **kwargs):
        kwargs.setdefault("gather_output", True)
        super().__init__(neox_args, input_size, output_size, bias=bias, **kwargs)


class TELayerNormMLP(nn.Module):
    """``norm(x) -> linear1 -> activation -> linear2`` with fp8 GEMMs; returns ``(output, bias)`` like the
    framework's MLP (the bias of the second linear is left for the caller's bias-dropout-add)."""

    def __init__(self, neox_args, init_method, output_layer_init_method, parallel_output=False,
                 multiple_of=256, MOE=False, MoE_mp_size=1, bias=True):
        super().__init__()
        from .norms import get_norm
        from .transformer import ParallelMLP
        a = _with(neox_args, te_layernorm_mlp=True)
        norm, eps = get_norm(a)
        self.norm = norm(a.hidden_size, eps=eps)
        self.mlp = ParallelMLP(neox_args=a, init_method=init_method, output_layer_init_method=output_layer_init_method,
                               parallel_output=parallel_output, multiple_of=multiple_of, MOE=MOE,
                               MoE_mp_size=MoE_mp_size)

    def forward(self, hidden_states):
        return self.mlp(self.norm(hidden_states))


class TEMultiheadAttention(nn.Module):
    def __init__(self, neox_args, attention_mask_func, init_method, output_layer_init_method, layer_number,
                 rpe=None, rotary=False, use_cache=False, parallel_output=False):
        super().__init__()
        from .transformer import ParallelSelfAttention
        self.attention = ParallelSelfAttention(
            neox_args=_with(neox_args, te_columnparallel=True, te_rowparallel=True),
            attention_mask_func=attention_mask_func, init_method=init_method,
            output_layer_init_method=output_layer_init_method, layer_number=layer_number, rpe=rpe, rotary=rotary,
            use_cache=use_cache, parallel_output=parallel_output)

    def forward(self, hidden_states, attention_mask, layer_past=None):
        return self.attention(hidden_states, attention_mask, layer_past=layer_past)


class TEDelayedScaling:
    def __init__(self, neox_args):
        if neox_args.te_fp8_format not in ("e4m3", "hybrid"):
            raise ValueError("E4M3 and HYBRID are the only supported FP8 formats.")
        self.neox_args = neox_args
        self.fp8_format = neox_args.te_fp8_format
        self.margin = neox_args.te_fp8_margin
        self.amax_compute_algo = neox_args.te_fp8_amax_compute_algo
        self.amax_history_len = neox_args.te_fp8_amax_history_len
        self.override_linear_precision = (False, False, not neox_args.te_fp8_wgrad)
        self.fp8_mha = neox_args.te_fp8_mha

    def linear_meta(self, device):
        """The per-linear scaling state this recipe describes."""
        from ..ops.fp8 import Fp8LinearMeta
        return Fp8LinearMeta.from_args(self.neox_args, device)

    def fp8_context(self):
        return contextlib.nullcontext()

    def get_context(self):
        return self.fp8_context()
