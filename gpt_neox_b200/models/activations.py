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


# ------------------------------------------------------------------ stand-alone GeLU entry points
def erf_gelu(x):
    """Exact GeLU, ``x * 0.5 * (1 + erf(x / sqrt(2)))`` (megatron/model/activations.py erf_gelu)."""
    return bias_act(x, None, "gelu")


def bias_gelu(bias, y):
    """tanh-approximated ``gelu(y + bias)`` (megatron/model/activations.py:85-95), one kernel on a GPU."""
    return bias_act(y, bias, "gelu_tanh")


def bias_gelu_back(g, bias, y):
    """Gradient of `bias_gelu` with respect to its pre-activation, given the output gradient ``g``."""
    import torch
    x = (y + bias).float()
    t = torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x))
    d = 0.5 * x * ((1 - t * t) * (0.79788456 + 0.1070322243 * x * x)) + 0.5 * (1 + t)
    return (d * g.float()).to(y.dtype)


class GeLUFunction:
    """``GeLUFunction.apply(input, bias)``: differentiable `bias_gelu`."""

    @staticmethod
    def apply(input, bias):
        return bias_gelu(bias, input)


class Gated_Activation:
    """Callable form of a gated activation: ``[value | gate] -> value * act(gate)`` (plus the bias first,
    when one is given), as megatron/model/transformer.py Gated_Activation."""

    def __init__(self, activation_name: str):
        if activation_name not in GATED:
            raise ValueError(f"{activation_name} is not a gated activation")
        self.name = activation_name

    def __call__(self, x, bias=None):
        if bias is not None:
            x = x + bias
        return gated_act(x, self.name)
