"""GPT2ModelPipe: the model as a flat list of layer specs.

Layer order and indices are the checkpoint contract (megatron/model/gpt2_model.py:183-343):
``0`` embedding, ``1`` transpose to [s,b,h], ``2..L+1`` blocks (transformer | gMLP | RWKV | Mamba),
``L+2`` transpose back, ``L+3`` final norm, ``L+4`` LM head (tied to the embedding through a
``TiedLayerSpec`` unless ``no_weight_tying``).  With ``pipe_parallel_size == 0`` the list is
flattened by ``to_sequential()``; otherwise each pipeline stage builds its contiguous slice and
``engine.pipeline`` drives it with a 1F1B schedule.
"""
from __future__ import annotations

import math
import re
from functools import partial

import torch
import torch.nn as nn

from .. import parallel as mpu
from .init_functions import get_init_methods
from .norms import get_norm
from .transformer import NormPipe, ParallelLinearPipe, ParallelTransformerLayerPipe, parallel_lm_logits
from .utils import Lambda, SequentialWrapper, recursive_setattr
from .word_embeddings import EmbeddingPipe, SoftEmbedding


class LayerSpec:
    """Deferred construction of a layer: only the owning pipeline stage instantiates it."""

    def __init__(self, typename, *module_args, **module_kwargs):
        self.typename, self.module_args, self.module_kwargs = typename, module_args, module_kwargs

    def build(self):
        return self.typename(*self.module_args, **self.module_kwargs)

    @property
    def name(self):
        return self.typename.__name__

    def __repr__(self):
        return f"LayerSpec({self.name})"


class TiedLayerSpec(LayerSpec):
    """A layer whose ``tied_weight_attr`` is shared with every other spec of the same ``key``."""

    def __init__(self, key, typename, *module_args, forward_fn=None, tied_weight_attr="weight", **module_kwargs):
        super().__init__(typename, *module_args, **module_kwargs)
        self.key, self.forward_fn, self.tied_weight_attr = key, forward_fn, tied_weight_attr


def gpt2_attention_mask_func(attention_scores, ltor_mask):
    mask_value = torch.finfo(attention_scores.dtype).min
    attention_scores.masked_fill_(ltor_mask, mask_value)
    return attention_scores


def cross_entropy(output, labels, _fp16=False):
    """Masked mean of the vocab-parallel per-token loss; ``labels = (labels, loss_mask)``
    (megatron/model/gpt2_model.py:60-78). The loss is computed from the bf16 / fp16 logits with fp32
    statistics: no fp32 copy of the logits is made."""
    labels, loss_mask = labels[0], labels[1]
    losses = mpu.vocab_parallel_cross_entropy(output.contiguous(), labels)
    loss_mask = loss_mask.view(-1)
    return torch.sum(losses.view(-1).float() * loss_mask) / loss_mask.sum()


def _pre_transformer_block(args):
    # [b, s, h] -> [s, b, h]; the mask rides along
    assert len(args) == 2, "Incorrect number of arguments to _pre_transformer_block"
    return args[0].transpose(0, 1).contiguous(), *args[1:]


def _post_transformer_block(args):
    assert len(args) == 2, "Incorrect number of arguments to _post_transformer_block"
    return args[0].transpose(0, 1).contiguous()


class GPT2ModelPipe(nn.Module):
    def __init__(self, neox_args, num_tokentypes=0, parallel_output=True, topology=None, use_cache=False):
        super().__init__()
        self.neox_args = neox_args
        self.use_cache = use_cache
        self.parallel_output = parallel_output
        self.hidden_size = neox_args.hidden_size
        self.num_tokentypes = num_tokentypes
        self.init_method, self.output_layer_init_method = get_init_methods(neox_args)
        self.__topology__ = topology
        self.loss_fn = partial(cross_entropy, _fp16=neox_args.fp16_lm_cross_entropy)
        self.activation_checkpoint_interval = neox_args.checkpoint_num_layers if neox_args.checkpoint_activations else 0
        self.specs = []
        self.init_specs()
        self.tied_modules = nn.ModuleDict()
        self.tied_specs = {}
        self._built = False
        self._local_start, self._local_stop = 0, len(self.specs)
        if neox_args.is_pipe_parallel:
            self._build_stage()

    # ------------------------------------------------------------------ specs
    def insert_layers(self, layers, idx):
        if isinstance(layers, nn.Module):
            self.specs.insert(idx, layers)
        elif isinstance(layers, (nn.ModuleList, nn.Sequential, list)):
            assert all(hasattr(l, "__call__") for l in layers), "all items in `layers` must be Callables"
            self.specs[idx:idx] = list(layers)
        else:
            raise ValueError(f"layer passed into {self.__class__.__name__}.insert_layer() should be either an "
                             f"nn.Module, an nn.ModuleList, an nn.Sequential object, or a list of callables "
                             f"not a {type(layers)}")
        if self._built:
            self._build_stage()

    def init_specs(self):
        a = self.neox_args
        weight_tying = not a.no_weight_tying
        self.specs = []
        emb_args = (a, self.hidden_size, a.padded_vocab_size, a.max_position_embeddings, a.hidden_dropout,
                    self.init_method, self.num_tokentypes)
        if weight_tying:
            self.specs.append(TiedLayerSpec("embed", EmbeddingPipe, *emb_args, tied_weight_attr="word_embeddings_weight"))
        else:
            self.specs.append(LayerSpec(EmbeddingPipe, *emb_args))
        self.specs.append(_pre_transformer_block)
        rpe_emb = None
        if a.pos_emb == "rpe":
            # T5 relative-position bias: ONE table per rank, shared by all of its attention layers
            # (megatron/model/gpt2_model.py:227-240)
            from ..parallel.layers import ParallelRelativePositionBias
            rpe_emb = ParallelRelativePositionBias(
                neox_args=a, scale=math.sqrt(a.hidden_size // a.num_attention_heads), causal=True,
                num_buckets=a.rpe_num_buckets, max_distance=a.rpe_max_distance, heads=a.num_attention_heads)
        for i in range(a.num_layers):
            layer_type = a.attention_config[i]
            if layer_type in ("gmlp", "amlp"):
                from .gmlp import GMLPBlock
                self.specs.append(LayerSpec(GMLPBlock, init_method=self.init_method, layer_number=i,
                                            output_layer_init_method=self.output_layer_init_method, neox_args=a,
                                            mask_fn=gpt2_attention_mask_func))
            elif layer_type == "rwkv":
                from .rwkv import RWKVResidualLayerPipe
                self.specs.append(LayerSpec(RWKVResidualLayerPipe, neox_args=a, layer_number=i))
            elif layer_type == "mamba":
                from .mamba import ParallelMambaResidualLayerPipe
                self.specs.append(LayerSpec(ParallelMambaResidualLayerPipe, neox_args=a, init_method=self.init_method,
                                            output_layer_init_method=self.output_layer_init_method, layer_number=i))
            else:
                self.specs.append(LayerSpec(ParallelTransformerLayerPipe, neox_args=a,
                                            attention_mask_func=gpt2_attention_mask_func,
                                            init_method=self.init_method,
                                            output_layer_init_method=self.output_layer_init_method, layer_number=i,
                                            rpe=rpe_emb, rotary=a.pos_emb == "rotary", use_cache=self.use_cache))
        self.specs.append(_post_transformer_block)
        norm, eps = get_norm(a)
        self.specs.append(LayerSpec(NormPipe, norm, a.hidden_size, eps=eps))

        def _logits_helper(embedding, lm_output):
            if a.use_mup:
                # MuReadout for the tied read-out: the embedding matrix grows with width in its fan-in
                lm_output = lm_output / embedding.word_embeddings.weight.infshape.width_mult()
            return parallel_lm_logits(lm_output, embedding.word_embeddings_weight, self.parallel_output,
                                      seq_parallel=a.sequence_parallel)

        if weight_tying:
            self.specs.append(TiedLayerSpec("embed", EmbeddingPipe, *emb_args, forward_fn=_logits_helper,
                                            tied_weight_attr="word_embeddings_weight"))
        else:
            self.specs.append(LayerSpec(ParallelLinearPipe, neox_args=a, init_method=self.init_method,
                                        parallel_output=self.parallel_output, is_last_layer=True))

    # ------------------------------------------------------------------ building
    def _seed_layer(self, idx):
        """With ``use_cpu_initialization`` every layer is drawn from its own seed, so the weights do
        not depend on how the layer list is cut into pipeline stages."""
        if getattr(self.neox_args, "use_cpu_initialization", False):
            torch.manual_seed(self.neox_args.seed * 1000 + idx)

    def _build_one(self, spec, idx):
        """-> (callable, module-or-None) for spec ``idx``."""
        self._seed_layer(idx)
        if isinstance(spec, TiedLayerSpec):
            # every owner of a tied module must start from the same weights: seed by its first occurrence
            first = next(i for i, sp in enumerate(self.specs) if getattr(sp, "key", None) == spec.key)
            self._seed_layer(first)
            if spec.key not in self.tied_modules:
                self.tied_modules[spec.key] = spec.build()
                self.tied_specs[spec.key] = spec
                if idx != first:
                    # a later pipeline stage's copy: the first owner counts it in the gradient norm
                    for p_ in self.tied_modules[spec.key].parameters():
                        p_._norm_skip = True
            mod = self.tied_modules[spec.key]
            if spec.forward_fn is not None:
                return partial(spec.forward_fn, mod), None
            return mod, None          # parameters live in tied_modules
        if isinstance(spec, LayerSpec):
            mod = spec.build()
            return mod, mod
        if isinstance(spec, nn.Module):
            return spec, spec
        return spec, None

    def partition_bounds(self, num_stages: int):
        """Stage boundaries over the spec list for ``pipe_partition_method``:
        ``type:<regex>`` balances the layers whose class name matches, ``parameters`` balances
        parameter counts, ``uniform`` balances the number of entries."""
        method = (self.neox_args.pipe_partition_method or "uniform").lower()
        n = len(self.specs)
        if method.startswith("type:"):
            pat = method.split(":", 1)[1]
            weights = [1 if re.search(pat, _spec_name(s), re.IGNORECASE) else 0 for s in self.specs]
        elif method == "parameters":
            weights = [_spec_param_count(s) for s in self.specs]
        else:
            weights = [1] * n
        return _balanced_partition(weights, num_stages)

    def _build_stage(self):
        pp = max(mpu.get_pipe_parallel_world_size(), 1)
        stage = mpu.get_pipe_parallel_rank()
        bounds = self.partition_bounds(pp)
        self._local_start, self._local_stop = bounds[stage], bounds[stage + 1]
        self.stage_bounds = bounds
        self.forward_funcs = []
        for idx in range(self._local_start, self._local_stop):
            fn, mod = self._build_one(self.specs[idx], idx)
            if mod is not None:
                self.add_module(str(idx), mod)
            self.forward_funcs.append(fn)
        self._built = True

    def is_first_stage(self):
        return self._local_start == 0

    def is_last_stage(self):
        return self._local_stop == len(self.specs)

    def forward_stage(self, x):
        """Run this stage's slice, with interval activation checkpointing."""
        interval = self.activation_checkpoint_interval
        funcs = self.forward_funcs
        if interval == 0:
            for f in funcs:
                x = f(x)
            return x
        i = 0
        names = ("ParallelTransformerLayerPipe", "GMLPBlock", "ParallelMambaResidualLayerPipe", "RWKVResidualLayerPipe")
        while i < len(funcs):
            chunk = funcs[i:i + interval]

            def run(*inputs, _chunk=chunk):
                y = inputs[0] if len(inputs) == 1 else inputs
                for f in _chunk:
                    y = f(y)
                return y
            if all(type(f).__name__ in names for f in chunk):
                x = mpu.checkpoint(run, *(x if isinstance(x, tuple) else (x,)))
            else:
                x = run(*(x if isinstance(x, tuple) else (x,)))
            i += interval
        return x

    def forward(self, forward_input):
        return self.forward_stage(forward_input)

    # ------------------------------------------------------------------ cache / modes
    def _set_parallel_output(self, value):
        final_layer = list(self.forward_funcs)[-1] if self._built else None
        if isinstance(final_layer, ParallelLinearPipe):
            final_layer.final_linear.set_parallel_output(value)
        self.parallel_output = value

    def inference_mode(self, use_cache=True):
        recursive_setattr(list(self.children()), "use_cache", use_cache, assert_type=bool)
        self._set_parallel_output(False)
        recursive_setattr(list(self.children()), "training", False)

    def train_mode(self):
        recursive_setattr(list(self.children()), "use_cache", False, assert_type=bool)
        self._set_parallel_output(True)
        recursive_setattr(list(self.children()), "training", True)

    def clear_cache(self):
        recursive_setattr(list(self.children()), "layer_past", None)

    # ------------------------------------------------------------------ sequential
    def to_sequential(self):
        """Flatten into a ``SequentialWrapper`` (used when ``pipe_parallel_size == 0``)."""
        layers = []
        tied_layers = {}
        for idx, spec in enumerate(self.specs):
            self._seed_layer(idx)
            if isinstance(spec, TiedLayerSpec):
                if spec.key in tied_layers:
                    layers.append(Lambda(partial(spec.forward_fn, tied_layers[spec.key][0])))
                else:
                    module = spec.build()
                    layers.append(module)
                    tied_layers.setdefault(spec.key, []).append(module)
            elif isinstance(spec, LayerSpec):
                layers.append(spec.build())
            elif hasattr(spec, "__call__"):
                layers.append(spec if isinstance(spec, nn.Module) else Lambda(spec))
            else:
                raise ValueError(f"Layer number {len(layers)} ({spec}) Not recognized")
        return SequentialWrapper(layers, self.activation_checkpoint_interval, mpu.checkpoint,
                                 parent_class_name=self.__class__.__name__)


def _spec_name(s):
    if isinstance(s, LayerSpec):
        return s.name
    if isinstance(s, nn.Module):
        return type(s).__name__
    return getattr(s, "__name__", "fn")


def _spec_param_count(s):
    if isinstance(s, nn.Module):
        return sum(p.numel() for p in s.parameters())
    if isinstance(s, LayerSpec):
        a = next((x for x in list(s.module_args) + list(s.module_kwargs.values()) if hasattr(x, "hidden_size")), None)
        if a is None:
            return 0
        h = a.hidden_size
        if s.name.startswith("Embedding") or s.name.startswith("ParallelLinear"):
            return a.padded_vocab_size * h
        if "Layer" in s.name or "Block" in s.name:
            return 12 * h * h
        return 2 * h
    return 0


def _balanced_partition(weights, parts):
    """Boundaries b[0..parts] minimising the heaviest part (prefix-sum binary search)."""
    n = len(weights)
    total = sum(weights)
    if total == 0:
        weights, total = [1] * n, n
    prefix = [0]
    for w in weights:
        prefix.append(prefix[-1] + w)

    def feasible(cap):
        bounds, start = [0], 0
        for _ in range(parts):
            end = start
            while end < n and prefix[end + 1] - prefix[start] <= cap:
                end += 1
            bounds.append(end)
            start = end
        return bounds if bounds[-1] == n else None

    lo, hi = max(weights), total
    best = feasible(hi)
    while lo < hi:
        mid = (lo + hi) // 2
        b = feasible(mid)
        if b is not None:
            best, hi = b, mid
        else:
            lo = mid + 1
    best = feasible(lo) or best
    # spread trailing zero-weight entries so no stage is empty when possible
    for i in range(1, parts):
        if best[i] <= best[i - 1] and best[i - 1] + 1 < n:
            best[i] = best[i - 1] + 1
    best[-1] = n
    return best
