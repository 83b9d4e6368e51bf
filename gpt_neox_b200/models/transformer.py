"""Transformer building blocks: ParallelMLP, ParallelLinear (LM head), ParallelSelfAttention,
ParallelTransformerLayer and their pipeline wrappers.

Module / parameter names and tensor layouts follow megatron/model/transformer.py:88-1248 (the
checkpoint contract: ``attention.query_key_value``, ``attention.dense``, ``mlp.linear1``,
``mlp.linear2``, ``input_layernorm``, ``post_attention_layernorm``; activations ``[s, b, h]``; fused
QKV rows grouped per head for MHA and ``[Q | K | V]`` for GQA).  The compute is organised around
this library's fused operators: QKV GEMM -> in-place partial rotary + flash attention on strided
views -> output GEMM with bias/residual epilogue; MLP as one autograd node with GeLU in the GEMM
epilogues; both LayerNorms of a GPT-J block from one pass over the input.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import parallel as mpu
from ..ops import fused as fused_ops
from ..ops.attention import flash_attention, next_dropout_seed
from ..ops.elementwise import bias_dropout_add
from ..ops.gemm import gemm as gemm_op
from ..ops.gemm import linear as linear_op
from ..ops.norm import dual_layer_norm
from ..ops.rope import apply_rotary
from ..ops.softmax import scaled_causal_softmax, scaled_masked_softmax
from ..parallel.mappings import (copy_to_model_parallel_region, gather_from_sequence_parallel_region,
                                 reduce_from_model_parallel_region,
                                 reduce_scatter_to_sequence_parallel_region)
from .activations import get_activation
from .norms import LayerNorm, RMSNorm, get_norm
from .positional_embeddings import AliBi, RotaryEmbedding


def get_parallel_linear(neox_args):
    """(column, row) linear classes.  The ``te_columnparallel`` / ``te_rowparallel`` / ``te_layernorm_mlp`` switches do
    not change the class: the parallel linears themselves run their GEMMs in fp8 then (per-tensor delayed scaling, or
    block scaling with ``te_fp8_recipe: mxfp8``; parallel/layers.py ``_fp8_or_bf16_linear``)."""
    return mpu.ColumnParallelLinear, mpu.RowParallelLinear


class ParallelMLP(nn.Module):
    """h -> ffn -> h with the hidden dimension sharded over the tensor-parallel group.

    ffn width (megatron/model/transformer.py:117-143): ``intermediate_size`` | ``expansion_factor*h``
    | ``4h``; gated activations use 2/3 of that, rounded up to ``mlp_multiple_of``, and linear1
    produces ``[value | gate]`` of twice the width."""

    def __init__(self, neox_args, init_method, output_layer_init_method, parallel_output=False,
                 multiple_of=256, MOE=False, MoE_mp_size=1):
        super().__init__()
        assert neox_args.intermediate_size is None or neox_args.expansion_factor is None
        self.activation_func, self.is_gated = get_activation(neox_args)
        self.activation_type = neox_args.activation
        self.bias_gelu_fusion = neox_args.bias_gelu_fusion
        self.multiple_of = multiple_of
        self.parallel_output = parallel_output
        self.sequence_parallel = bool(neox_args.sequence_parallel) and mpu.get_model_parallel_world_size() > 1
        self.recompute_act = False
        if neox_args.intermediate_size:
            ffn_dim = neox_args.intermediate_size
        elif neox_args.expansion_factor:
            ffn_dim = int(neox_args.expansion_factor * neox_args.hidden_size)
        else:
            ffn_dim = 4 * neox_args.hidden_size
        ffn_dim_in = ffn_dim
        if self.is_gated:
            ffn_dim = int(ffn_dim * 2 / 3) if not neox_args.intermediate_size else ffn_dim
            m = neox_args.mlp_multiple_of
            ffn_dim = m * ((ffn_dim + m - 1) // m)
            ffn_dim_in = ffn_dim
            ffn_dim = 2 * ffn_dim
        Column, Row = get_parallel_linear(neox_args)
        self.linear1 = Column(neox_args=neox_args, input_size=neox_args.hidden_size, output_size=ffn_dim,
                              gather_output=False, init_method=init_method, skip_bias_add=True,
                              bias=neox_args.use_bias_in_mlp)
        self.linear2 = Row(neox_args=neox_args, input_size=ffn_dim_in, output_size=neox_args.hidden_size,
                           input_is_parallel=True, init_method=output_layer_init_method,
                           parallel_output=parallel_output, skip_bias_add=True,
                           bias=neox_args.use_bias_in_mlp)

    def _fusable(self, x):
        if getattr(self.linear1, "use_fp8", False) or getattr(self.linear2, "use_fp8", False):
            return False        # fp8 GEMMs run through the per-module path
        return (not self.is_gated) and self.activation_type == "gelu" and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)

    def forward(self, hidden_states, residual=None, out_bias=None):
        """-> (output without linear2's bias, that bias). ``residual`` (optional, fused path only)
        is added inside the second GEMM's epilogue; so is ``out_bias`` (a bias vector that already
        includes linear2's: the returned bias is then None)."""
        if self._fusable(hidden_states):
            if self.sequence_parallel:
                x = gather_from_sequence_parallel_region(hidden_states, seq_dim=0)
            else:
                x = copy_to_model_parallel_region(hidden_states)
            kind = "tanh" if self.bias_gelu_fusion else "erf"
            out = fused_ops.mlp_gelu(x, self.linear1.weight, self.linear1.bias, self.linear2.weight, out_bias,
                                     residual=residual, kind=kind, recompute_act=self.recompute_act)
            if not self.parallel_output:
                if self.sequence_parallel:
                    out = reduce_scatter_to_sequence_parallel_region(out, seq_dim=0)
                else:
                    out = reduce_from_model_parallel_region(out)
            return out, (None if out_bias is not None else self.linear2.bias)
        assert residual is None and out_bias is None
        intermediate, bias = self.linear1(hidden_states)
        if self.is_gated:
            if bias is not None:
                intermediate = intermediate + bias
            intermediate = self.activation_func(intermediate)
        else:
            intermediate = self.activation_func(intermediate, bias)
        return self.linear2(intermediate)


class ParallelLinear(nn.Module):
    """Final (LM-head) projection, column-parallel over the vocabulary; no bias
    (megatron/model/transformer.py:201-265)."""

    def __init__(self, neox_args, parallel_output=True, init_method=nn.init.xavier_normal_, is_last_layer=False):
        super().__init__()
        self.is_rm = neox_args.train_impl == "rm"
        parallelism = neox_args.output_layer_parallelism if not self.is_rm else "row"
        if parallelism == "column":
            self.final_linear = mpu.ColumnParallelLinear(
                neox_args=neox_args, input_size=neox_args.hidden_size, output_size=neox_args.padded_vocab_size,
                bias=False, init_method=init_method, gather_output=not parallel_output, skip_bias_add=False,
                mup_rescale_parameters=is_last_layer, seq_dim=1)
        elif not self.is_rm:
            raise NotImplementedError("row parallelism of the output layer is not supported")
        else:  # reward model: scalar head
            self.rm_linear = mpu.RowParallelLinear(
                neox_args=neox_args, input_size=neox_args.hidden_size, output_size=1, bias=False,
                input_is_parallel=False, init_method=init_method, parallel_output=False, skip_bias_add=False)

    def forward(self, hidden_states):
        if not self.is_rm:
            return self.final_linear(hidden_states)
        return self.rm_linear(hidden_states)


class ParallelSelfAttention(nn.Module):
    """Multi-head / grouped-query self-attention, heads sharded over the tensor-parallel group."""

    def __init__(self, neox_args, attention_mask_func, init_method, output_layer_init_method, layer_number,
                 rpe=None, rotary=False, use_cache=False, parallel_output=False):
        super().__init__()
        Column, Row = get_parallel_linear(neox_args)
        self.fp16 = neox_args.precision == "fp16"
        self.bf16 = neox_args.precision == "bfloat16"
        self.attention_mask_func = attention_mask_func
        self.apply_query_key_layer_scaling = neox_args.apply_query_key_layer_scaling
        self.use_cache = use_cache
        self.attention_softmax_in_fp32 = neox_args.attention_softmax_in_fp32 or self.apply_query_key_layer_scaling
        self.layer_number = layer_number
        ws = mpu.get_model_parallel_world_size()
        self.hidden_size_per_partition = mpu.divide(neox_args.hidden_size, ws)
        self.hidden_size_per_attention_head = mpu.divide(neox_args.hidden_size, neox_args.num_attention_heads)
        self.num_attention_heads_per_partition = mpu.divide(neox_args.num_attention_heads, ws)
        self.pos_emb = neox_args.pos_emb
        self.use_qk_layernorm = neox_args.use_qk_layernorm
        if self.use_qk_layernorm:
            norm, eps = get_norm(neox_args)
            self.qk_layernorm = norm([self.num_attention_heads_per_partition, self.hidden_size_per_attention_head],
                                     eps=eps)
        self.sliding_window_width = neox_args.sliding_window_width
        self.gqa = bool(neox_args.num_kv_heads) and neox_args.num_kv_heads != neox_args.num_attention_heads
        if self.gqa:
            self.num_kv_heads_per_partition = mpu.divide(neox_args.num_kv_heads, ws)
            self.kv_hidden_size = neox_args.num_kv_heads * self.hidden_size_per_attention_head
        else:
            self.num_kv_heads_per_partition = self.num_attention_heads_per_partition
            self.kv_hidden_size = neox_args.hidden_size
        self.query_key_value = Column(neox_args=neox_args, input_size=neox_args.hidden_size,
                                      output_size=neox_args.hidden_size + 2 * self.kv_hidden_size,
                                      gather_output=False, init_method=init_method,
                                      bias=neox_args.use_bias_in_attn_linear)
        coeff = None
        self.norm_factor = math.sqrt(self.hidden_size_per_attention_head)
        if self.apply_query_key_layer_scaling:
            coeff = max(1, self.layer_number)
            self.norm_factor *= coeff
        if neox_args.use_mup:
            self.norm_factor = self.hidden_size_per_attention_head
        self.coeff = coeff
        # net softmax scale of the flash kernels: 1 / sqrt(d) (query-key layer scaling cancels out), 1 / d under muP
        self.attn_scale = 1.0 / self.hidden_size_per_attention_head if neox_args.use_mup \
            else 1.0 / math.sqrt(self.hidden_size_per_attention_head)
        self.rpe = rpe
        if self.pos_emb == "alibi":
            self.alibi_embed = AliBi(neox_args.num_attention_heads, ws, mpu.get_model_parallel_rank())
        if rotary:
            if neox_args.rotary_pct == 1:
                self.rotary_ndims = None
            else:
                assert neox_args.rotary_pct < 1
                self.rotary_ndims = int(self.hidden_size_per_attention_head * neox_args.rotary_pct)
            dim = self.rotary_ndims if self.rotary_ndims is not None else self.hidden_size_per_attention_head
            self.rotary_emb = RotaryEmbedding(dim, base=neox_args.rotary_emb_base,
                                              max_seq_len=neox_args.seq_length, precision=neox_args.params_dtype,
                                              save_inv_freqs=neox_args.rotary_save_freqs_buffer)
            self.rotary_dim = dim
        else:
            self.rotary_emb = None
            self.rotary_dim = 0
        self.rope_fusion = neox_args.rope_fusion
        self.attention_type = neox_args.attention_config[layer_number]
        self.use_flash_attention = self.attention_type == "flash"
        self.sparse = self.attention_type not in ("global", "flash")
        self.sparse_layout = None
        if self.sparse:
            # block-sparse pattern: on the GPU the flash kernels take the block layout (key tiles without a live
            # block are skipped); the token mask serves the masked-softmax path (CPU, relative-position bias,
            # block sizes the kernels do not take)
            from ..ops.attention import BlockLayout
            from .sparse_attention import block_layout, token_mask
            cfg = neox_args.sparsity_config or {}
            self.register_buffer("sparse_mask", token_mask(self.attention_type, neox_args.seq_length, cfg,
                                                           seed=layer_number), persistent=False)
            block = cfg.get("block", 16)
            nb = (neox_args.seq_length + block - 1) // block
            self.sparse_layout = BlockLayout(block_layout(self.attention_type, nb, cfg, seed=layer_number), block)
        self.dropout_p = neox_args.attention_dropout
        self.attention_dropout = nn.Dropout(self.dropout_p)
        self.dense = Row(neox_args=neox_args, input_size=neox_args.hidden_size,
                         output_size=neox_args.hidden_size, input_is_parallel=True,
                         init_method=output_layer_init_method, skip_bias_add=True,
                         parallel_output=parallel_output, bias=neox_args.use_bias_in_attn_linear)

    # -------------------------------------------------------------------- helpers
    def _split_qkv(self, mixed):
        sq, b = mixed.shape[0], mixed.shape[1]
        np_, kvp, hn = self.num_attention_heads_per_partition, self.num_kv_heads_per_partition, \
            self.hidden_size_per_attention_head
        return fused_ops._qkv_views(mixed, np_, kvp, hn)

    def _global_attention(self, q, k, v, attention_mask):
        """Unfused path: scores -> (+rpe / +alibi) -> scaled masked softmax -> dropout -> context.
        q [sq,b,np,hn], k/v [sk,b,np,hn] -> [sq, b, np*hn]."""
        sq, b, np_, hn = q.shape
        sk = k.shape[0]
        if k.shape[2] != np_:  # GQA without flash: repeat kv heads
            rep = np_ // k.shape[2]
            k = k.repeat_interleave(rep, dim=2)
            v = v.repeat_interleave(rep, dim=2)
        q2 = q.reshape(sq, b * np_, hn).transpose(0, 1)
        k2 = k.reshape(sk, b * np_, hn).transpose(0, 1)
        scores = torch.bmm(q2, k2.transpose(1, 2))                      # [b*np, sq, sk]
        scale = 1.0 / self.norm_factor
        plain_causal = self.rpe is None and self.pos_emb != "alibi" and self.sliding_window_width is None \
            and attention_mask is None
        if self.coeff is not None:
            scale_softmax = self.coeff
            scores = scores * scale
        else:
            scale_softmax = None
        if plain_causal:
            probs = scaled_causal_softmax(scores.contiguous(), scale if scale_softmax is None else scale_softmax)
        else:
            s4 = scores.view(b, np_, sq, sk)
            if scale_softmax is None:
                s4 = s4 * scale
            if self.rpe is not None:
                s4 = s4 + self.rpe(sq, sk).to(s4.dtype)
            if self.pos_emb == "alibi":
                s4 = self.alibi_embed(s4)
            mask = attention_mask
            if mask is not None and (mask.shape[-2] != sq or mask.shape[-1] != sk):
                if mask.shape[-2] >= sk and mask.shape[-1] >= sk:
                    mask = mask[..., sk - sq:sk, :sk]    # decoding with a KV cache: rows of the new positions
                else:
                    # a mask built for the new tokens only (pipeline stages build it from the step's input):
                    # the causal / sliding-window mask over the cached keys is derived from positions below
                    mask = None
            if mask is None:
                qpos = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
                kpos = torch.arange(sk, device=q.device)[None, :]
                mask = kpos > qpos
                if self.sliding_window_width is not None:
                    mask = mask | (kpos < qpos - self.sliding_window_width)
                mask = mask[None, None]
            probs = scaled_masked_softmax(s4.contiguous(), mask, scale_softmax or 1.0).view(b * np_, sq, sk)
        if self.dropout_p > 0 and self.training:
            with mpu.get_cuda_rng_tracker().fork():
                probs = self.attention_dropout(probs)
        v2 = v.reshape(sk, b * np_, hn).transpose(0, 1)
        ctx = torch.bmm(probs.to(v2.dtype), v2)                          # [b*np, sq, hn]
        return ctx.view(b, np_, sq, hn).permute(2, 0, 1, 3).reshape(sq, b, np_ * hn)

    # -------------------------------------------------------------------- forward
    def forward(self, hidden_states, attention_mask=None, layer_past=None, residual=None):
        """hidden_states [sq, b, h] -> (output [sq, b, h] without dense bias, dense bias)
        (+ the updated KV cache when ``use_cache``)."""
        mixed, _ = self.query_key_value(hidden_states)
        np_, kvp, hn = self.num_attention_heads_per_partition, self.num_kv_heads_per_partition, \
            self.hidden_size_per_attention_head
        has_past = layer_past is not None and (not torch.is_tensor(layer_past) or layer_past.numel() > 0)
        simple = (self.use_flash_attention and not self.use_cache and not has_past and not self.use_qk_layernorm
                  and self.rpe is None)
        # attention dropout runs inside the flash kernels (mask regenerated in the backward); every
        # tensor-parallel rank draws its own seed stream, as its heads are different heads
        drop_p = self.dropout_p if self.training else 0.0
        drop_seed = next_dropout_seed(mpu.get_model_parallel_rank()) if drop_p > 0 else None
        cos = sin = None
        if self.rotary_emb is not None:
            cos, sin = self.rotary_emb(seq_len=mixed.shape[0] + (layer_past[0].shape[0] if has_past else 0))
        if simple:
            ctx = fused_ops.qkv_attention(
                mixed, num_heads=np_, num_kv_heads=kvp, head_dim=hn, rotary_dim=self.rotary_dim, cos=cos, sin=sin,
                scale=self.attn_scale,
                window=self.sliding_window_width if self.sliding_window_width is not None else -1,
                alibi=self.alibi_embed.slopes if self.pos_emb == "alibi" else None, dropout_p=drop_p, seed=drop_seed)
            present = None
        else:
            q, k, v = self._split_qkv(mixed)
            if self.use_qk_layernorm:
                q = self.qk_layernorm(q.contiguous())
                k = self.qk_layernorm(k.contiguous()) if kvp == np_ else k
            offset = layer_past[0].shape[0] if has_past else 0
            if self.rotary_emb is not None:
                q = apply_rotary(q, cos, sin, self.rotary_dim, offset)
                k = apply_rotary(k, cos, sin, self.rotary_dim, offset)
            if has_past:
                k = torch.cat((layer_past[0].type_as(k), k), dim=0)
                v = torch.cat((layer_past[1].type_as(v), v), dim=0)
            present = torch.stack((k, v)) if self.use_cache else None
            sparse_kernel = (self.sparse and self.rpe is None and q.is_cuda and self.sparse_layout.kernel_ok
                             and q.dtype in (torch.bfloat16, torch.float16) and hn % 8 == 0 and hn <= 128)
            if (self.use_flash_attention and self.rpe is None) or sparse_kernel:
                o = flash_attention(q.permute(1, 0, 2, 3), k.permute(1, 0, 2, 3), v.permute(1, 0, 2, 3),
                                    causal=True, scale=self.attn_scale,
                                    window=self.sliding_window_width if self.sliding_window_width is not None else -1,
                                    alibi=self.alibi_embed.slopes if self.pos_emb == "alibi" else None,
                                    dropout_p=drop_p, seed=drop_seed,
                                    block_layout=self.sparse_layout if sparse_kernel else None)
                ctx = o.permute(1, 0, 2, 3).reshape(q.shape[0], q.shape[1], np_ * hn)
            else:
                mask = attention_mask if not self.use_flash_attention else None
                if self.sparse:
                    sk_ = k.shape[0]
                    mask = self.sparse_mask[..., sk_ - q.shape[0]:sk_, :sk_]
                ctx = self._global_attention(q, k, v, mask)
        # output projection; bias (and the optional residual) are applied by the caller / epilogue
        if residual is not None and ctx.is_cuda and not self.dense.sequence_parallel and \
                mpu.get_model_parallel_world_size() == 1:
            out = _linear_residual(ctx, self.dense.weight, residual)
            bias = self.dense.bias
        else:
            out, bias = self.dense(ctx)
            if residual is not None:
                out = out + residual
        if self.use_cache:
            return out, bias, present
        return out, bias


class _LinearResidualFn(torch.autograd.Function):
    """y = x @ W^T + residual with the add in the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, w, residual):
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, residual.shape[-1])
        y = gemm_op(x2.contiguous() if not x2.is_contiguous() else x2, w,
                    residual=r2.contiguous() if not r2.is_contiguous() else r2)
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        from ..ops.gemm import wgrad
        x2, w = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        gx = gemm_op(gy2, w, trans_b=True).view(ctx.x_shape)
        gw = wgrad(gy2, x2, w)
        return gx, gw, gy2.view(gy.shape)


def _linear_residual(x, w, residual):
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16):
        return _LinearResidualFn.apply(x, w, residual)
    return F.linear(x, w) + residual


class ParallelTransformerLayer(nn.Module):
    """One transformer block [s, b, h] -> [s, b, h]: GPT-J parallel residual
    (``x + attn(ln1(x)) + mlp(ln2(x))``, one tensor-parallel reduction per block) or the sequential
    pre-LN form; MoE FFN on layers selected by ``moe_expert_interval``."""

    def __init__(self, neox_args, attention_mask_func, init_method, output_layer_init_method, layer_number,
                 rpe=None, rotary=False, use_cache=False):
        super().__init__()
        self.layer_number = layer_number
        self.neox_args = neox_args
        norm, eps = get_norm(neox_args)
        self.input_layernorm = norm(neox_args.hidden_size, eps=eps)
        self.use_cache = use_cache
        self.hidden_dropout = neox_args.hidden_dropout
        self.bias_dropout_fusion = neox_args.bias_dropout_fusion
        self.gpt_j_residual = neox_args.gpt_j_residual
        self.gpt_j_tied = neox_args.gpt_j_tied
        self.mlp_type = neox_args.activation
        self.moe_type = None
        self.num_experts = neox_args.moe_num_experts if (neox_args.moe_num_experts > 1 and
                                                          layer_number % neox_args.moe_expert_interval == 0) else 1
        ws = mpu.get_model_parallel_world_size()
        self.sequence_parallel = bool(neox_args.sequence_parallel) and ws > 1
        if self.gpt_j_residual:
            if self.sequence_parallel:
                self.reduce = lambda t: reduce_scatter_to_sequence_parallel_region(t, seq_dim=0)
            else:
                self.reduce = reduce_from_model_parallel_region
        self.attention = ParallelSelfAttention(
            neox_args=neox_args, attention_mask_func=attention_mask_func, init_method=init_method,
            output_layer_init_method=output_layer_init_method, layer_number=layer_number, rpe=rpe,
            use_cache=self.use_cache, rotary=rotary, parallel_output=self.gpt_j_residual)
        if not (self.gpt_j_residual and self.gpt_j_tied):
            self.post_attention_layernorm = norm(neox_args.hidden_size, eps=eps)
        if self.num_experts <= 1:
            self.mlp = ParallelMLP(neox_args=neox_args, init_method=init_method,
                                   output_layer_init_method=output_layer_init_method,
                                   parallel_output=self.gpt_j_residual,
                                   multiple_of=neox_args.mlp_multiple_of)
        else:
            from .moe import ParallelDroplessMoE
            self.mlp = ParallelDroplessMoE(neox_args=neox_args, init_method=init_method,
                                           output_layer_init_method=output_layer_init_method)
        self.layer_past = None

    def _dual_norm_ok(self, x):
        return (isinstance(self.input_layernorm, LayerNorm) and not self.gpt_j_tied
                and len(self.input_layernorm.normalized_shape) == 1)

    def forward(self, x, attention_mask=None, layer_past=None):
        layer_past = layer_past if layer_past is not None else self.layer_past
        p = self.hidden_dropout if self.training else 0.0
        ws = mpu.get_model_parallel_world_size()
        if self.gpt_j_residual:
            residual = x
            if self.gpt_j_tied:
                x1 = x2 = self.input_layernorm(x)
            elif self._dual_norm_ok(x):
                # the residual stream rides through the norm node: its gradient joins the two norm
                # gradients inside one backward kernel
                residual, x1, x2 = dual_layer_norm(x, self.input_layernorm.weight, self.input_layernorm.bias,
                                                   self.post_attention_layernorm.weight,
                                                   self.post_attention_layernorm.bias, self.input_layernorm.eps,
                                                   carry=True)
            else:
                x1, x2 = self.input_layernorm(x), self.post_attention_layernorm(x)
            fusable = (p == 0.0 and x.is_cuda and self.num_experts <= 1 and not self.use_cache
                       and isinstance(self.mlp, ParallelMLP) and self.mlp._fusable(x2))
            fast = fusable and ws == 1
            if fusable and self.sequence_parallel:
                from ..ops import fused_tp
                be = fused_tp.backend(x, mpu.get_model_parallel_group())
                m_full = x.shape[0] * x.shape[1] * ws
                if be is not None and be.can_fuse(m_full, x.shape[-1], x.shape[-1]) and \
                        be.can_fuse(m_full, x.shape[-1], self.mlp.linear1.output_size_per_partition):
                    # Tensor + sequence parallel block with every collective inside a GEMM kernel:
                    # QKV and MLP-up gather their input shards in front of the GEMM; the attention
                    # output stays a partial sum and rides as a residual of the MLP-down GEMM, whose
                    # epilogue does the block's single reduce-scatter, then adds biases and x.
                    attn_partial, b_attn = self.attention(x1, attention_mask, layer_past=layer_past)
                    b_mlp = self.mlp.linear2.bias
                    bias_total = _sum_bias(b_attn, b_mlp)
                    if bias_total is not None:
                        bias_total = bias_total * ws      # added on every rank before the reduction
                    kind = "tanh" if self.mlp.bias_gelu_fusion else "erf"
                    return fused_tp.mlp_gelu_sp(x2, self.mlp.linear1.weight, self.mlp.linear1.bias,
                                                self.mlp.linear2.weight, attn_partial, bias_total, residual, kind, be)
            if fast:
                # x + attn + b_attn + mlp + b_mlp with both adds of matrices inside GEMM epilogues:
                #   t = dense(ctx) + x ;  out = linear2(h) + t ; the two bias vectors are added once.
                t, b_attn = self.attention(x1, attention_mask, layer_past=layer_past, residual=residual)
                out, _ = self.mlp(x2, residual=t, out_bias=_sum_bias(b_attn, self.mlp.linear2.bias))
                return out
            att = self.attention(x1, attention_mask, layer_past=layer_past)
            if self.use_cache:
                attention_output, attention_bias, presents = att
                self.layer_past = presents
            else:
                attention_output, attention_bias = att
            attention_output = bias_dropout_add(attention_output, attention_bias, None, p, self.training)
            if self.num_experts > 1:
                # the MoE layer returns one complete tensor (no bias, nothing left to sum over the tensor-parallel
                # group), so only the attention branch goes through the reduction.  (The reference unpacks two
                # values here and cannot run this combination, megatron/model/transformer.py:1103.)
                moe_output = self.mlp(x2)
                return residual + (self.reduce(attention_output) if ws > 1 else attention_output) + moe_output
            mlp_output, mlp_bias = self.mlp(x2)
            output = bias_dropout_add(mlp_output, mlp_bias, attention_output, p, self.training)
            # one reduction for both branches (all-reduce, or reduce-scatter under sequence parallelism)
            return residual + (self.reduce(output) if ws > 1 else output)
        # sequential residual form
        if (isinstance(self.input_layernorm, LayerNorm) and len(self.input_layernorm.normalized_shape) == 1) \
                or isinstance(self.input_layernorm, RMSNorm):
            residual, ln_out = self.input_layernorm(x, carry=True)
        else:
            residual, ln_out = x, self.input_layernorm(x)
        att = self.attention(ln_out, attention_mask, layer_past=layer_past)
        if self.use_cache:
            attention_output, attention_bias, presents = att
            self.layer_past = presents
        else:
            attention_output, attention_bias = att
        attention_output = bias_dropout_add(attention_output, attention_bias, residual, p, self.training)
        layernorm_output = self.post_attention_layernorm(attention_output)
        mlp_bias = None
        if self.num_experts <= 1:
            mlp_output, mlp_bias = self.mlp(layernorm_output)
        else:
            mlp_output = self.mlp(layernorm_output)
        if mlp_bias is None and (self.num_experts > 1 or p == 0.0):
            return mlp_output + attention_output
        return bias_dropout_add(mlp_output, mlp_bias, attention_output, p, self.training)


def _sum_bias(a, b):
    if a is None:
        return b
    if b is None:
        return a
    return a + b


class ParallelTransformerLayerPipe(ParallelTransformerLayer):
    """Pipeline form: ``(hidden_states, attention_mask)`` in and out."""

    def forward(self, args):
        assert len(args) == 2, "ParallelTransformerLayerPipe expects 2 arguments - hidden_states and attention_mask"
        hidden_states, attention_mask = args
        return super().forward(hidden_states, attention_mask), attention_mask


class ParallelLinearPipe(ParallelLinear):
    def forward(self, args):
        assert isinstance(args, torch.Tensor), "ParallelLinearPipe expects a single argument - hidden_states"
        logits, _bias = super().forward(args)
        return logits


class NormPipe(nn.Module):
    def __init__(self, norm_class, hidden_size, eps):
        super().__init__()
        self.norm = norm_class(hidden_size, eps=eps)

    def forward(self, args):
        assert not isinstance(args, tuple), "NormPipe should only receive a single tensor as input"
        return self.norm(args)


def parallel_lm_logits(input_, word_embeddings_weight, parallel_output, seq_parallel=False, seq_dim=1, bias=None):
    """Logits against a (tied) vocabulary-sharded embedding matrix
    (megatron/model/transformer.py:1218-1248)."""
    if seq_parallel:
        input_parallel = gather_from_sequence_parallel_region(input_, seq_dim=seq_dim)
    else:
        input_parallel = copy_to_model_parallel_region(input_)
    logits_parallel = linear_op(input_parallel, word_embeddings_weight, bias)
    if parallel_output:
        return logits_parallel
    return mpu.gather_from_model_parallel_region(logits_parallel)
