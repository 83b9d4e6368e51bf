"""Rotary embedding under the reference's fused entry points (megatron/model/fused_rope.py:58-140).

``t`` is ``[s, b, heads, d]``; ``freqs`` ``[s, 1, 1, d2]`` holds the angles with both halves equal
(``cat(f, f)``), ``cos_`` / ``sin_`` are their cosine / sine.  The first ``d2`` features of every head are
rotated (halves paired: feature i with i + d2/2), the rest pass through.  Runs `ops.rope.apply_rotary`: the
vectorised kernel on a GPU for bf16, PyTorch otherwise."""
from __future__ import annotations

import torch

from ..ops.rope import apply_rotary


def _finish(out, transpose_output_memory):
    if transpose_output_memory:          # memory laid out [b, s, ...] behind the same [s, b, ...] view
        out = out.transpose(0, 1).contiguous().transpose(0, 1)
    return out


def fused_apply_rotary_pos_emb_cached(t: torch.Tensor, cos_: torch.Tensor, sin_: torch.Tensor,
                                      transpose_output_memory: bool = False) -> torch.Tensor:
    d2 = cos_.shape[-1]
    half = d2 // 2
    cos = cos_.reshape(cos_.shape[0], d2)[:, :half].float().contiguous()
    sin = sin_.reshape(sin_.shape[0], d2)[:, :half].float().contiguous()
    return _finish(apply_rotary(t, cos, sin, d2, 0), transpose_output_memory)


def fused_apply_rotary_pos_emb(t: torch.Tensor, freqs: torch.Tensor, transpose_output_memory: bool = False) -> torch.Tensor:
    f = freqs.float()
    return fused_apply_rotary_pos_emb_cached(t, torch.cos(f), torch.sin(f), transpose_output_memory)


class FusedRoPEFunc:
    """``FusedRoPEFunc.apply(t, freqs, transpose_output_memory)`` (differentiable)."""
    apply = staticmethod(fused_apply_rotary_pos_emb)


class FusedRoPECachedFunc:
    """``FusedRoPECachedFunc.apply(t, cos_, sin_, transpose_output_memory)`` (differentiable)."""
    apply = staticmethod(fused_apply_rotary_pos_emb_cached)
