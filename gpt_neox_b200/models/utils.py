"""Model utilities (megatron/model/utils.py): weight-decay parameter groups, the sequential
wrapper with interval activation checkpointing and curriculum truncation, sequence-parallel norm
gradient sync, ``recursive_setattr``."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import parallel as mpu
from ..parallel.random import checkpoint
from .norms import LayerNorm, NonParametricLayernorm, RMSNorm, ScaleNorm

_NORM_TYPES = (LayerNorm, RMSNorm, ScaleNorm, NonParametricLayernorm, nn.LayerNorm)


def get_fusion_type(neox_args):
    """The softmax fusion the configuration asks for (megatron/model/utils.py:364-370)."""
    from .fused_softmax import SoftmaxFusionTypes
    if neox_args.scaled_upper_triang_masked_softmax_fusion:
        return SoftmaxFusionTypes.upper_triang
    if neox_args.scaled_masked_softmax_fusion:
        return SoftmaxFusionTypes.general
    return SoftmaxFusionTypes.none


def get_params_for_weight_decay_optimization(module, neox_args):
    """Two groups: decayed, and not decayed (every parameter of a norm module, every ``bias``, every
    parameter flagged ``_no_weight_decay``). With ``weight_decay == 0`` a single group."""
    decay = {"params": [], "name": "weight_decay_params"}
    no_decay = {"params": [], "weight_decay": 0.0, "name": "no_weight_decay_params"}

    def is_no_decay_module(m):
        return isinstance(m, _NORM_TYPES) or type(m).__name__ in ("MixedFusedLayerNorm", "MixedFusedRMSNorm")

    for m in module.modules():
        if is_no_decay_module(m) or neox_args.weight_decay == 0.0:
            no_decay["params"].extend([p for p in m._parameters.values() if p is not None and p.requires_grad])
        else:
            for n, p in m._parameters.items():
                if p is None or not p.requires_grad:
                    continue
                if n == "bias" or getattr(p, "_no_weight_decay", False):
                    no_decay["params"].append(p)
                else:
                    decay["params"].append(p)
    if neox_args.weight_decay == 0.0:
        return [no_decay]
    return [decay, no_decay]


def exists(x):
    return x is not None


class Lambda(nn.Module):
    def __init__(self, func):
        super().__init__()
        self.func = func

    def forward(self, x):
        return self.func(x)


class SequentialWrapper(nn.Module):
    """Runs the flattened layer list; checkpoints every ``activation_checkpoint_interval`` layers of
    the checkpointable kinds; truncates the batch to ``curriculum_seqlen`` when curriculum learning
    is active (megatron/model/utils.py:90-229)."""

    def __init__(self, layers, activation_checkpoint_interval, activation_checkpoint_func, parent_class_name=None):
        super().__init__()
        self.sequential = nn.Sequential(*layers)
        self.activation_checkpoint_interval = activation_checkpoint_interval
        self.parent_class_name = parent_class_name
        self.activation_checkpoint_func = activation_checkpoint_func
        self.batch_fn = None

    def _is_checkpointable(self, funcs):
        names = ("ParallelTransformerLayerPipe", "GMLPBlock", "ParallelMambaResidualLayerPipe", "RWKVResidualLayerPipe")
        if self.parent_class_name == "GPT2ModelPipe":
            return all(type(f).__name__ in names for f in funcs)
        return any(len(list(f.parameters())) > 0 for f in funcs if isinstance(f, nn.Module))

    def set_batch_fn(self, fn):
        self.batch_fn = fn

    def inference_mode(self, use_cache=True):
        _set_use_cache(self.sequential, use_cache)
        recursive_setattr(self.sequential, "training", False)

    def train_mode(self):
        _set_use_cache(self.sequential, False)
        recursive_setattr(self.sequential, "training", True)

    def clear_cache(self):
        recursive_setattr(self.sequential, "layer_past", None)

    def forward(self, forward_input, curriculum_seqlen=None, labels=None, neox_args=None):
        if self.batch_fn:
            forward_input = self.batch_fn(forward_input)
        if curriculum_seqlen is not None and isinstance(forward_input, tuple) and len(forward_input) == 3:
            neox_args.update_value("curriculum_seqlen", curriculum_seqlen)
            tokens, position_ids, attention_mask = forward_input
            if curriculum_seqlen < tokens.size(1):
                tokens = tokens[:, :curriculum_seqlen].contiguous()
                position_ids = position_ids[:, :curriculum_seqlen].contiguous()
                if labels is not None:
                    labels = labels[:, :curriculum_seqlen].contiguous()
                if attention_mask is not None:
                    attention_mask = attention_mask[:, :, :curriculum_seqlen, :curriculum_seqlen].contiguous()
            forward_input = (tokens, position_ids, attention_mask)

        def exec_range_func(start, end):
            def exec_func(*inputs):
                if len(inputs) == 1:
                    inputs = inputs[0]
                for layer in self.sequential[start:end]:
                    inputs = layer(inputs)
                return inputs
            return exec_func

        n = len(self.sequential)
        if self.activation_checkpoint_interval == 0:
            x = exec_range_func(0, n)(forward_input)
        else:
            x = forward_input
            start = 0
            while start < n:
                end = min(start + self.activation_checkpoint_interval, n)
                funcs = self.sequential[start:end]
                if not isinstance(x, tuple):
                    x = (x,)
                if self._is_checkpointable(funcs):
                    x = self.activation_checkpoint_func(exec_range_func(start, end), *x)
                else:
                    x = exec_range_func(start, end)(*x)
                start = end
        return x

    def clear_layer_past(self):
        self.clear_cache()


def recursive_setattr(m, attr, value, assert_type=None, type_filter=None):
    """Set ``attr`` on every submodule that already has it."""
    if assert_type is not None:
        assert isinstance(value, assert_type), "Value is not the correct type."
    if isinstance(m, (list, nn.ModuleList, nn.Sequential)):
        for i in m:
            recursive_setattr(i, attr, value, assert_type, type_filter)
    elif isinstance(m, nn.Module):
        if hasattr(m, attr) and (type_filter is None or isinstance(m, type_filter)):
            setattr(m, attr, value)
        for c in m.children():
            recursive_setattr(c, attr, value, assert_type, type_filter)


def _set_use_cache(modules, value: bool):
    recursive_setattr(modules, "use_cache", value, assert_type=bool)


def configure_sparse_attention(neox_args, attention_type, num_attention_heads, mpu_):
    """-> bool token mask [1, 1, seq, seq] (True = masked) of the block-sparse pattern (megatron/model/utils.py:261-361;
    the reference returns a DeepSpeed SparseSelfAttention module, here the pattern feeds the masked-softmax path)."""
    from .sparse_attention import token_mask
    return token_mask(attention_type, neox_args.seq_length, neox_args.sparsity_config or {})

def reduce_weight_grads_from_model_parallel_region(input_):
    """All-reduce a gradient over the tensor-parallel group (norm weights under sequence
    parallelism see only their sequence shard)."""
    if mpu.get_model_parallel_world_size() == 1:
        return input_
    from ..comm.collectives import all_reduce
    dt = input_.dtype
    if mpu.get_fp32_allreduce() and dt != torch.float32:
        input_ = input_.float()
    input_ = all_reduce(input_.contiguous(), group=mpu.get_model_parallel_group())
    return input_.to(dt)


def mark_norms_for_sequence_parallel_grad_sync(module, neox_args):
    """Under sequence parallelism, flag every norm parameter so the engine sums its gradient over
    the tensor-parallel group (one flat all-reduce per step instead of one hook per parameter,
    megatron/model/utils.py:373-412)."""
    if not neox_args.sequence_parallel:
        return
    for name, m in module.named_modules():
        if name.endswith("qk_layernorm"):
            # normalises this rank's heads of the FULL sequence (the QKV projection gathered it): its
            # parameters are per partition and their gradients complete; summing them over the group would
            # mix the partitions (the reference flags them by name and does, megatron/model/utils.py:398-412)
            continue
        if "norm" in name.lower() or isinstance(m, _NORM_TYPES):
            for p in m.parameters(recurse=False):
                if p.requires_grad:
                    p.sequence_parallel_grad_sync = True
        # MoE routers and experts are replicated over the tensor-parallel group (expert parallelism is a
        # separate axis here) and, under sequence parallelism, see only this rank's part of the sequence
        elif type(m).__name__ == "ParallelDroplessMoE":
            for p in m.parameters(recurse=True):
                if p.requires_grad and not getattr(p, "model_parallel", False):
                    p.sequence_parallel_grad_sync = True


def get_parallel_linear(neox_args):
    from .transformer import get_parallel_linear as g
    return g(neox_args)
