"""Activation selector (megatron/model/activations.py:27-75). Returns ``(fn, is_gated)`` where for
plain activations ``fn(x, bias=None)`` computes ``act(x + bias)`` and for gated ones ``fn(x)`` takes
``[value | gate]`` and returns ``value * act(gate)``."""
from __future__ import annotations

from ..ops.elementwise import GATED, bias_act, gated_act


def get_activation(neox_args):
    name = neox_args.activation
    if name in GATED:
        return (lambda x: gated_act(x, name)), True
    if name == "gelu":
        if neox_args.onnx_safe and neox_args.bias_gelu_fusion:
            raise ValueError("onnx_safe + bias_gelu_fusion not compatible")
        # the tanh approximation only with bias_gelu_fusion, exact erf otherwise
        kind = "gelu_tanh" if neox_args.bias_gelu_fusion else "gelu"
        return (lambda x, bias=None: bias_act(x, bias, kind)), False
    if name in ("relu", "softsign", "swish", "mish", "silu"):
        return (lambda x, bias=None: bias_act(x, bias, name)), False
    raise ValueError(f"Activation function {name} not recognized")
