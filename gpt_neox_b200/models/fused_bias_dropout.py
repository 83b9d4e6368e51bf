"""``dropout(x + bias) + residual`` under the reference's names (megatron/model/fused_bias_dropout.py:28-57).

Every entry point lands in `ops.elementwise.bias_dropout_add`: on a GPU one kernel adds the bias, applies
Philox dropout and adds the residual in a single pass and regenerates the mask in backward; on CPU the
PyTorch statement of the same function runs.  ``bias`` and ``residual`` may be None.
"""
from __future__ import annotations

from ..ops.elementwise import bias_dropout_add as _kernel


def bias_dropout_add(x, bias, residual, prob: float, training: bool):
    """``residual + dropout(x + bias, prob)``; dropout is the identity when ``training`` is false."""
    return _kernel(x, bias, residual, prob, training)


def _bound_to(training: bool, name: str):
    def fn(x, bias, residual, prob):
        return _kernel(x, bias, residual, prob, training)
    fn.__name__ = fn.__qualname__ = name
    fn.__doc__ = f"`bias_dropout_add` with training={training}."
    return fn


#: the two pre-bound forms the transformer layer picks between
bias_dropout_add_fused_train = _bound_to(True, "bias_dropout_add_fused_train")
bias_dropout_add_fused_inference = _bound_to(False, "bias_dropout_add_fused_inference")


def get_bias_dropout_add(training: bool):
    """The four-argument form ``(x, bias, residual, prob)`` for the given mode."""
    return bias_dropout_add_fused_train if training else bias_dropout_add_fused_inference
