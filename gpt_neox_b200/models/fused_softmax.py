"""Scale + mask + softmax module with the reference's surface (megatron/model/fused_softmax.py:24-204).

``FusedScaleMaskSoftmax(input_in_fp16, input_in_bf16, fusion_type, mask_func, softmax_in_fp32, scale)``
takes scores ``[b, np, sq, sk]`` and an optional boolean mask (True = masked out).  On a GPU with bf16
scores the two fusion types run this library's softmax kernels (`ops.softmax`), which have no limit on the
key length; otherwise (CPU, fp32 / fp16 scores, ``SoftmaxFusionTypes.none``) the PyTorch statement of the
same function runs.
"""
from __future__ import annotations

import enum

import torch
import torch.nn as nn

from ..ops import softmax as softmax_ops


class SoftmaxFusionTypes(enum.Enum):
    upper_triang = 1    # causal mask built inside the kernel
    general = 2         # mask given by the caller
    none = 3            # plain PyTorch


class ScaledUpperTriangMaskedSoftmax:
    """``apply(inputs [attn_batches, sq, sk], scale)``: scale, causal mask, softmax."""

    @staticmethod
    def apply(inputs, scale):
        return softmax_ops.scaled_causal_softmax(inputs, float(scale))


class ScaledMaskedSoftmax:
    """``apply(inputs [b, np, sq, sk], mask [b or 1, 1, sq, sk], scale)``: scale, mask, softmax."""

    @staticmethod
    def apply(inputs, mask, scale):
        return softmax_ops.scaled_masked_softmax(inputs, mask, float(scale))


class FusedScaleMaskSoftmax(nn.Module):
    def __init__(self, input_in_fp16, input_in_bf16, fusion_type, mask_func, softmax_in_fp32, scale):
        super().__init__()
        if not isinstance(fusion_type, SoftmaxFusionTypes):
            raise AssertionError(f"Invalid fusion type {fusion_type}")
        if scale is not None and not softmax_in_fp32:
            raise AssertionError("softmax should be in fp32 when scaled")
        self.input_in_fp16, self.input_in_bf16 = bool(input_in_fp16), bool(input_in_bf16)
        self.input_in_float16 = self.input_in_fp16 or self.input_in_bf16
        self.upper_triang_mask_fusion = fusion_type == SoftmaxFusionTypes.upper_triang
        self.general_mask_fusion = fusion_type == SoftmaxFusionTypes.general
        self.fusion = fusion_type != SoftmaxFusionTypes.none
        self.mask_func, self.softmax_in_fp32, self.scale = mask_func, softmax_in_fp32, scale

    def is_kernel_available(self, mask, b, np, sq, sk):
        """The kernels take any ``sk``; they need a fusion type, and a mask when the type is ``general``."""
        if not self.fusion:
            return False
        if self.upper_triang_mask_fusion:
            return sq == sk
        return mask is not None

    def forward(self, input, mask):
        assert input.dim() == 4, "scores are [b, np, sq, sk]"
        if self.is_kernel_available(mask, *input.size()):
            return self.forward_fused_softmax(input, mask)
        return self.forward_torch_softmax(input, mask)

    def forward_fused_softmax(self, input, mask):
        b, np, sq, sk = input.size()
        scale = 1.0 if self.scale is None else self.scale
        if self.upper_triang_mask_fusion:
            assert sq == sk, "causal mask is only for self attention"
            return ScaledUpperTriangMaskedSoftmax.apply(input.reshape(-1, sq, sk), scale).view(b, np, sq, sk)
        return ScaledMaskedSoftmax.apply(input, mask, scale)

    def forward_torch_softmax(self, input, mask):
        x = input.float() if (self.input_in_float16 and self.softmax_in_fp32) else input
        if self.scale is not None:
            x = x * self.scale
        if mask is not None:
            x = self.mask_func(x, mask)
        probs = torch.softmax(x, dim=-1)
        if self.input_in_float16 and self.softmax_in_fp32:
            probs = probs.half() if self.input_in_fp16 else probs.bfloat16()
        return probs

    @staticmethod
    def get_batch_per_block(sq, sk, b, np):
        return softmax_ops.get_batch_per_block(sq, sk, b, np)
