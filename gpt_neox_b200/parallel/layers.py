"""Tensor-parallel layers: VocabParallelEmbedding, ColumnParallelLinear, RowParallelLinear,
ParallelRelativePositionBias.

Same constructor / forward contracts as megatron/mpu/layers.py:98-790 (weights ``[out/p, in]`` for
column, ``[out, in/p]`` for row; forward returns ``(output, bias_if_skipped)``).  The matmuls run
on this library's tcgen05 GEMM; under tensor parallelism the collective next to each GEMM is
issued through ``comm`` (NCCL in baseline mode, in-kernel NVLink paths in fused mode).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.parameter import Parameter

from ..ops.embedding import embedding as embedding_op
from ..ops.gemm import linear as linear_op
from . import state as mpu
from .mappings import (copy_to_model_parallel_region, gather_from_model_parallel_region,
                       gather_from_sequence_parallel_region, reduce_from_model_parallel_region,
                       reduce_scatter_to_sequence_parallel_region, scatter_to_model_parallel_region,
                       scatter_to_sequence_parallel_region)
from .random import get_cuda_rng_tracker
from .utils import VocabUtility, divide


def _fused_backend(x):
    """Symmetric-memory backend of the tensor-parallel group when the fused communication mode
    applies to ``x`` (CUDA bf16), else None."""
    from ..ops.fused_tp import backend
    return backend(x, mpu.get_model_parallel_group())


def _device(neox_args):
    if getattr(neox_args, "use_cpu_initialization", False) or not torch.cuda.is_available():
        return torch.device("cpu")
    return torch.device("cuda", torch.cuda.current_device())


def _fp8_or_bf16_linear(mod, x, weight, bias):
    """The module's GEMM: fp8 tensor cores when the module was built with fp8 enabled (``te_columnparallel`` /
    ``te_rowparallel`` / ``te_layernorm_mlp``), the bf16 kernel otherwise."""
    if getattr(mod, "use_fp8", False) and x.is_cuda and getattr(mod._fp8_args, "te_fp8_recipe", "delayed") == "mxfp8" \
            and (x.numel() // x.shape[-1]) % 32 == 0 and weight.shape[0] % 32 == 0 and weight.shape[1] % 32 == 0:
        # block-scaled recipe: one power-of-two scale per 32 elements, no amax history (ops/fp8.py mxfp8_linear)
        from ..ops.fp8 import mxfp8_linear
        return mxfp8_linear(x, weight, bias, hybrid=getattr(mod._fp8_args, "te_fp8_format", "hybrid") == "hybrid")
    if getattr(mod, "use_fp8", False) and x.is_cuda and x.dtype == torch.bfloat16 and \
            (x.numel() // x.shape[-1]) % 8 == 0 and weight.shape[0] % 16 == 0 and weight.shape[1] % 16 == 0:
        from ..ops.fp8 import Fp8LinearMeta, fp8_linear
        if mod.fp8_meta is None:
            mod.fp8_meta = Fp8LinearMeta.from_args(mod._fp8_args, x.device)
        return fp8_linear(x, weight, bias, mod.fp8_meta)
    return linear_op(x, weight, bias)


def _set_tp_attrs(p, is_parallel, dim, stride):
    p.model_parallel = is_parallel
    p.partition_dim = dim
    p.partition_stride = stride


def _init_partitioned(weight, full_shape, partition_dim, init_method, neox_args, stride=1):
    """Initialise this rank's shard. With ``use_cpu_initialization`` the full matrix is drawn once
    (identical on all ranks) and sliced, so a tensor-parallel model starts from exactly the
    weights of the unsharded one; otherwise the shard is drawn directly from the per-rank
    model-parallel RNG stream (megatron/mpu/layers.py:44-95)."""
    ws = mpu.get_model_parallel_world_size()
    _set_tp_attrs(weight, True, partition_dim, stride)
    if not getattr(neox_args, "use_cpu_initialization", False):
        with get_cuda_rng_tracker().fork():
            init_method(weight)
        return
    master = torch.empty(full_shape, dtype=torch.float32)
    init_method(master)
    per = full_shape[partition_dim] // ws
    shard = master.narrow(partition_dim, mpu.get_model_parallel_rank() * per, per)
    with torch.no_grad():
        weight.copy_(shard.to(weight.dtype))


class VocabParallelEmbedding(nn.Module):
    """Embedding with the vocabulary dimension sharded over the tensor-parallel group."""

    def __init__(self, neox_args, num_embeddings, embedding_dim, init_method=nn.init.xavier_normal_):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.model_parallel_size = mpu.get_model_parallel_world_size()
        self.vocab_start_index, self.vocab_end_index = VocabUtility.vocab_range_from_global_vocab_size(
            num_embeddings, mpu.get_model_parallel_rank(), self.model_parallel_size)
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.init_method = init_method
        self.use_mup = getattr(neox_args, "use_mup", False)
        self.mup_embedding_mult = getattr(neox_args, "mup_embedding_mult", 1.0)
        self.weight = Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim,
                                            device=_device(neox_args), dtype=neox_args.params_dtype))
        _init_partitioned(self.weight, (num_embeddings, embedding_dim), 0, init_method, neox_args)

    def forward(self, input_, to_sequence_parallel=False):
        """``to_sequence_parallel``: return this rank's slice along the sequence (dim 1) instead of the whole
        [batch, seq, hidden] result."""
        if self.model_parallel_size > 1 and input_.is_cuda and input_.dim() == 2:
            # over peer memory the owner of a vocabulary entry stores its row straight into the output of the
            # rank(s) that need it: no all-reduce over rows of zeros, no separate scatter
            from ..ops import fused_tp
            be = fused_tp.backend(self.weight, mpu.get_model_parallel_group())
            if be is not None and be.can_embed_push(input_, self.weight, to_sequence_parallel):
                out = _EmbedPushFn.apply(input_, self.weight, self.vocab_start_index, be, bool(to_sequence_parallel))
                return out * self.mup_embedding_mult if self.use_mup else out
        out = embedding_op(input_, self.weight, self.vocab_start_index)
        if self.use_mup:
            out = out * self.mup_embedding_mult
        if self.model_parallel_size > 1:
            out = reduce_from_model_parallel_region(out)
            if to_sequence_parallel:
                out = scatter_to_sequence_parallel_region(out, seq_dim=1)
        return out


class _EmbedPushFn(torch.autograd.Function):
    """Vocabulary-parallel lookup whose rows travel straight to their consumers (comm/symm.py embed_push).  Backward:
    the gradient rows of all tokens (gathered along the sequence if the output was a slice) are scattered into this
    rank's part of the table by the kernel the unfused path uses."""

    @staticmethod
    def forward(ctx, ids, table, vocab_start, be, sp):
        ctx.save_for_backward(ids)
        ctx.table, ctx.vocab_start, ctx.sp = table, int(vocab_start), sp
        return be.embed_push(ids, table, vocab_start, sp)

    @staticmethod
    def backward(ctx, gy):
        from ..ops import _lib
        from ..ops.gemm import LAUNCHES
        from .mappings import _gather_along_seq_dim
        (ids,) = ctx.saved_tensors
        table = ctx.table
        V, H = table.shape
        g = _gather_along_seq_dim(gy.contiguous(), 1) if ctx.sp else gy
        g2 = g.reshape(-1, H).contiguous()
        flat = ids.reshape(-1).contiguous()
        mg = getattr(table, "main_grad", None)
        target = mg if mg is not None else torch.zeros((V, H), device=table.device, dtype=torch.float32)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(g2).nx_embedding_bwd(_lib.ptr(flat), _lib.ptr(g2), _lib.ptr(target), flat.numel(), H,
                                                 ctx.vocab_start, V, _lib.stream()), "nx_embedding_bwd")
        return None, (None if mg is not None else target.to(table.dtype)), None, None, None


class ParallelRelativePositionBias(nn.Module):
    """T5 relative-position bias with heads sharded over the tensor-parallel group
    (megatron/mpu/layers.py:215-380)."""

    def __init__(self, neox_args, scale, causal=True, num_buckets=32, max_distance=128, heads=8,
                 init_method=nn.init.xavier_normal_):
        super().__init__()
        self.scale, self.causal, self.num_buckets, self.max_distance, self.heads = \
            scale, causal, num_buckets, max_distance, heads
        ws = mpu.get_model_parallel_world_size()
        self.head_start_index, self.head_end_index = VocabUtility.vocab_range_from_global_vocab_size(
            heads, mpu.get_model_parallel_rank(), ws)
        self.num_heads_per_partition = self.head_end_index - self.head_start_index
        self.weight = Parameter(torch.empty(num_buckets, self.num_heads_per_partition,
                                            device=_device(neox_args), dtype=neox_args.params_dtype))
        _init_partitioned(self.weight, (num_buckets, heads), 1, init_method, neox_args)
        self._q_len_cached = self._k_len_cached = self._rel_pos_bucket_cached = None

    @staticmethod
    def get_heads_range(global_n_heads, rank, world_size):
        per = divide(global_n_heads, world_size)
        return rank * per, (rank + 1) * per

    def _relative_position_bucket(self, relative_position, num_buckets=32, max_distance=128):
        ret = 0
        n = -relative_position
        if not self.causal:
            num_buckets //= 2
            ret += (n < 0).long() * num_buckets
            n = torch.abs(n)
        else:
            n = torch.max(n, torch.zeros_like(n))
        max_exact = num_buckets // 2
        is_small = n < max_exact
        val_if_large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) /
                                    math.log(max_distance / max_exact) * (num_buckets - max_exact)).long()
        val_if_large = torch.min(val_if_large, torch.full_like(val_if_large, num_buckets - 1))
        return ret + torch.where(is_small, n, val_if_large)

    def compute_bias(self, q_len, k_len):
        dev = self.weight.device
        # the queries are the LAST q_len positions of the keys (incremental decoding: one query at k_len - 1)
        q_pos = torch.arange(k_len - q_len, k_len, dtype=torch.long, device=dev)
        k_pos = torch.arange(k_len, dtype=torch.long, device=dev)
        rel = k_pos[None, :] - q_pos[:, None]
        bucket = self._relative_position_bucket(rel, self.num_buckets, self.max_distance)
        values = F.embedding(bucket, self.weight)          # [q, k, heads/p]
        return values.permute(2, 0, 1).unsqueeze(0) * self.scale

    def forward(self, q_len, k_len):
        return self.compute_bias(q_len, k_len)


class ColumnParallelLinear(nn.Module):
    """Y = X A^T + b with A sharded along its output dimension: A_i is ``[out/p, in]``.

    Forward: (sequence-parallel: all-gather X along ``seq_dim`` | else identity with an all-reduce
    in backward) -> GEMM -> optional all-gather of the output."""

    def __init__(self, neox_args, input_size, output_size, bias=True, gather_output=True,
                 init_method=nn.init.xavier_normal_, stride=1, keep_master_weight_for_test=False,
                 skip_bias_add=False, mup_rescale_parameters=False, seq_dim=0):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.gather_output, self.skip_bias_add = gather_output, skip_bias_add
        self.use_fp8 = bool(getattr(neox_args, "te_columnparallel", False) or getattr(neox_args, "te_layernorm_mlp", False))
        self.fp8_meta, self._fp8_args = None, neox_args
        ws = mpu.get_model_parallel_world_size()
        self.output_size_per_partition = divide(output_size, ws)
        self.sequence_parallel = bool(neox_args.sequence_parallel) and ws > 1
        self.seq_dim = seq_dim
        self.init_method, self.stride = init_method, stride
        self.mup_rescale_parameters = mup_rescale_parameters
        self.use_mup = getattr(neox_args, "use_mup", False)
        self.width_mult_value = 1.0
        dev, dt = _device(neox_args), neox_args.params_dtype
        self.weight = Parameter(torch.empty(self.output_size_per_partition, input_size, device=dev, dtype=dt))
        _init_partitioned(self.weight, (output_size, input_size), 0, init_method, neox_args, stride)
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size_per_partition, device=dev, dtype=dt))
            _set_tp_attrs(self.bias, True, 0, stride)
        else:
            self.register_parameter("bias", None)

    def width_mult(self):
        return self.width_mult_value

    def set_parallel_output(self, value: bool):
        assert isinstance(value, bool)
        self.gather_output = not value

    def forward(self, input_):
        if self.use_mup and self.mup_rescale_parameters:
            input_ = input_ / self.width_mult()
        bias = self.bias if not self.skip_bias_add else None
        be = _fused_backend(input_) if (self.sequence_parallel and self.seq_dim == 0) else None
        if be is not None and be.can_fuse(input_.numel() // input_.shape[-1] * be.ws, self.input_size,
                                          self.output_size_per_partition):
            # all-gather of the sequence shards fused into the GEMM (peer stores over NVLink)
            from ..ops.fused_tp import ag_linear
            output_parallel = ag_linear(input_, self.weight, bias, be)
        else:
            if self.sequence_parallel:
                input_parallel = gather_from_sequence_parallel_region(input_, seq_dim=self.seq_dim)
            else:
                input_parallel = copy_to_model_parallel_region(input_)
            output_parallel = _fp8_or_bf16_linear(self, input_parallel, self.weight, bias)
        output = gather_from_model_parallel_region(output_parallel) if self.gather_output else output_parallel
        return output, (self.bias if self.skip_bias_add else None)


class RowParallelLinear(nn.Module):
    """Y = X A^T + b with A sharded along its input dimension: A_i is ``[out, in/p]``.

    Forward: (optional scatter of X) -> GEMM -> sequence-parallel reduce-scatter | all-reduce |
    nothing when ``parallel_output`` (the caller reduces, e.g. once per GPT-J block) -> + bias."""

    def __init__(self, neox_args, input_size, output_size, bias=True, input_is_parallel=False,
                 init_method=nn.init.xavier_normal_, stride=1, keep_master_weight_for_test=False,
                 skip_bias_add=False, parallel_output=False, mup_rescale_parameters=False, seq_dim=0):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.input_is_parallel, self.skip_bias_add = input_is_parallel, skip_bias_add
        self.use_fp8 = bool(getattr(neox_args, "te_rowparallel", False) or getattr(neox_args, "te_layernorm_mlp", False))
        self.fp8_meta, self._fp8_args = None, neox_args
        self.parallel_output = parallel_output
        ws = mpu.get_model_parallel_world_size()
        self.input_size_per_partition = divide(input_size, ws)
        self.sequence_parallel = bool(neox_args.sequence_parallel) and ws > 1
        self.seq_dim = seq_dim
        self.init_method, self.stride = init_method, stride
        self.mup_rescale_parameters = mup_rescale_parameters
        self.use_mup = getattr(neox_args, "use_mup", False)
        self.width_mult_value = 1.0
        dev, dt = _device(neox_args), neox_args.params_dtype
        self.weight = Parameter(torch.empty(output_size, self.input_size_per_partition, device=dev, dtype=dt))
        _init_partitioned(self.weight, (output_size, input_size), 1, init_method, neox_args, stride)
        if bias:
            self.bias = Parameter(torch.zeros(output_size, device=dev, dtype=dt))
            if self.sequence_parallel and not parallel_output:
                # added after the reduce-scatter: each rank sees only its sequence shard, so the
                # gradient of this replicated bias is summed over the tensor-parallel group
                self.bias.sequence_parallel_grad_sync = True
        else:
            self.register_parameter("bias", None)

    def width_mult(self):
        return self.width_mult_value

    def set_parallel_output(self, parallel_output: bool):
        assert isinstance(parallel_output, bool)
        self.parallel_output = parallel_output

    def forward(self, input_):
        if self.use_mup and self.mup_rescale_parameters:
            input_ = input_ / self.width_mult()
        input_parallel = input_ if self.input_is_parallel else scatter_to_model_parallel_region(input_)
        be = _fused_backend(input_parallel) if (self.sequence_parallel and not self.parallel_output
                                                and self.seq_dim == 0) else None
        if be is not None and be.can_fuse(input_parallel.numel() // input_parallel.shape[-1],
                                          self.input_size_per_partition, self.output_size):
            # reduce-scatter fused into the GEMM epilogue; a bias that is not skipped is added after it
            from ..ops.fused_tp import linear_rs
            b = self.bias if not self.skip_bias_add else None
            out = linear_rs(input_parallel, self.weight, b, None, be)
            return out, (self.bias if self.skip_bias_add else None)
        if not self.sequence_parallel and not self.parallel_output and mpu.get_model_parallel_world_size() > 1 \
                and not getattr(self, "use_fp8", False):
            be = _fused_backend(input_parallel)
            rows = input_parallel.numel() // input_parallel.shape[-1]
            if be is not None and be.can_fuse_ar(rows, self.input_size_per_partition, self.output_size):
                # all-reduce fused into the GEMM (reduce-scatter in the epilogue + owner broadcast over NVLink)
                from ..ops.fused_tp import linear_ar
                b = self.bias if not self.skip_bias_add else None
                return linear_ar(input_parallel, self.weight, b, be), (self.bias if self.skip_bias_add else None)
        output_parallel = _fp8_or_bf16_linear(self, input_parallel, self.weight, None)
        if self.sequence_parallel and not self.parallel_output:
            output_ = reduce_scatter_to_sequence_parallel_region(output_parallel, seq_dim=self.seq_dim)
        elif not self.parallel_output:
            output_ = reduce_from_model_parallel_region(output_parallel)
        else:
            output_ = output_parallel
        if not self.skip_bias_add:
            return (output_ + self.bias if self.bias is not None else output_), None
        return output_, self.bias
