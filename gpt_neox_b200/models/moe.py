"""Dropless mixture-of-experts FFN (megatron/model/moe.py:25-250) with expert parallelism decoupled
from tensor parallelism.

Token flow per layer: route (top-k) -> sort the T*k routed copies by expert -> **all-to-all dispatch**
over the expert-parallel group (each rank owns ``experts / ep`` experts) -> regroup received rows by
local expert -> grouped expert MLP -> **all-to-all combine** back to the source ranks -> weighted sum of
the k copies.  On CUDA bf16 (GeLU experts) both exchanges run as peer loads inside the permutation
kernels (ops/moe_ep.py); the NCCL / gloo all-to-all below is the general path.  The reference instead replicates all tokens on every tensor-parallel rank, slices the
local experts' rows and variable-size all-gathers the outputs (moe.py:85-160,
mpu/mappings.py:147-183); with EP = 1 both degenerate to the same local computation.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import parallel as mpu
from .moe_mlp import ParallelGroupedLLaMAMLP, ParallelGroupedMLP
from .router import SinkhornRouter, TopKTokenChoiceRouter


class _AllToAllRows(torch.autograd.Function):
    """Variable-size all-to-all of rows; backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, send_sizes, recv_sizes, group):
        ctx.send_sizes, ctx.recv_sizes, ctx.group = send_sizes, recv_sizes, group
        out = x.new_empty((sum(recv_sizes),) + tuple(x.shape[1:]))
        _a2a(out, x.contiguous(), recv_sizes, send_sizes, group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send_sizes),) + tuple(g.shape[1:]))
        _a2a(out, g.contiguous(), ctx.send_sizes, ctx.recv_sizes, ctx.group)
        return out, None, None, None


def _a2a(out, inp, out_sizes, in_sizes, group):
    if dist.get_backend(group) == "gloo":
        # gloo has no all_to_all: exchange through all_gather of padded blocks (test path only)
        ws = dist.get_world_size(group)
        me = dist.get_rank(group)
        sizes_t = torch.tensor(in_sizes, dtype=torch.long)
        all_sizes = [torch.empty_like(sizes_t) for _ in range(ws)]
        dist.all_gather(all_sizes, sizes_t, group=group)
        mx = int(max(int(s.sum()) for s in all_sizes))
        pad = inp.new_zeros((mx,) + tuple(inp.shape[1:]))
        pad[: inp.shape[0]] = inp
        bufs = [torch.empty_like(pad) for _ in range(ws)]
        dist.all_gather(bufs, pad, group=group)
        pieces = []
        for src in range(ws):
            off = int(all_sizes[src][:me].sum())
            pieces.append(bufs[src][off: off + int(all_sizes[src][me])])
        out.copy_(torch.cat(pieces, dim=0))
    else:
        dist.all_to_all_single(out, inp, output_split_sizes=list(out_sizes), input_split_sizes=list(in_sizes),
                               group=group)


class ParallelDroplessMLP(nn.Module):
    """Permute, dispatch, expert MLP, combine, un-permute."""

    def __init__(self, neox_args, init_method, output_layer_init_method):
        super().__init__()
        self.num_experts = neox_args.moe_num_experts
        self.top_k = neox_args.moe_top_k
        self.ep_size = mpu.get_expert_parallel_world_size()
        self.experts_per_rank = self.num_experts // self.ep_size
        gated = neox_args.activation in ("swiglu", "geglu", "reglu", "bilinear", "glu")
        mlp_cls = ParallelGroupedLLaMAMLP if gated else ParallelGroupedMLP
        self.mlp = mlp_cls(neox_args=neox_args, init_method=init_method,
                           output_layer_init_method=output_layer_init_method)
        self.gated = gated
        self.use_kernels = True        # device-side plan / permute / grouped GEMM path (CUDA bf16, EP = 1)
        self.bias_gelu_fusion = bool(neox_args.bias_gelu_fusion)

    def indices_and_bins(self, top_expert):
        """Sort routed copies by expert: (sorted expert ids, permutation, tokens per expert)."""
        flat = top_expert.reshape(-1)
        bin_ids, indices = torch.sort(flat, stable=True)
        tokens_per_expert = torch.bincount(flat, minlength=self.num_experts)
        return indices, bin_ids, tokens_per_expert

    def forward(self, x, expert_weights, expert_indices):
        """x [s, b, h]; expert_weights / indices [s*b, k] -> [s, b, h]."""
        in_shape = x.shape
        x2 = x.reshape(-1, x.shape[-1])
        T, k = expert_indices.shape
        if (self.use_kernels and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and self.ep_size == 1 and not self.gated
                and self.mlp.activation_type == "gelu" and x2.shape[1] % 8 == 0
                and self.mlp.per_expert_ff_dim % 8 == 0):
            from ..ops.moe import experts_gelu
            out = experts_gelu(x2.contiguous(), expert_weights, expert_indices, self.mlp.w1, self.mlp.w2,
                               self.num_experts, "tanh" if self.bias_gelu_fusion else "erf")
            return out.view(in_shape)
        if (self.use_kernels and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and self.ep_size > 1 and not self.gated
                and self.mlp.activation_type == "gelu" and x2.shape[1] % 8 == 0 and self.top_k <= 8
                and self.mlp.per_expert_ff_dim % 8 == 0):
            from ..ops import moe_ep
            group = mpu.get_expert_parallel_group()
            if moe_ep.enabled() and dist.get_backend(group) == "nccl":
                # dispatch and combine as peer loads inside the permutation kernels: no NCCL all-to-all
                # and no host read of the per-expert counts
                out = moe_ep.experts_gelu_ep(x2.contiguous(), expert_weights, expert_indices, self.mlp.w1,
                                             self.mlp.w2, self.num_experts, group,
                                             "tanh" if self.bias_gelu_fusion else "erf")
                return out.view(in_shape)
        indices, _bin_ids, tpe = self.indices_and_bins(expert_indices)
        token_of_copy = torch.div(indices, k, rounding_mode="floor")
        routed = x2.index_select(0, token_of_copy)                      # expert-sorted copies
        if self.ep_size > 1:
            group = mpu.get_expert_parallel_group()
            counts = tpe.view(self.ep_size, self.experts_per_rank)
            # counts every rank sends me, per (source rank, local expert)
            recv_counts = torch.empty_like(counts)
            if dist.get_backend(group) == "gloo":
                allc = [torch.empty_like(counts) for _ in range(self.ep_size)]
                dist.all_gather(allc, counts.contiguous(), group=group)
                me = dist.get_rank(group)
                recv_counts = torch.stack([c[me] for c in allc])
            else:
                dist.all_to_all_single(recv_counts, counts.contiguous(), group=group)
            send_sizes = counts.sum(1).tolist()
            recv_mat = recv_counts.tolist()
            recv_sizes = [sum(r) for r in recv_mat]
            got = _AllToAllRows.apply(routed, send_sizes, recv_sizes, group)   # grouped by (src, expert)
            # regroup by local expert
            order, off = [], 0
            starts = []
            for r in recv_mat:
                row = []
                for n in r:
                    row.append(off)
                    off += n
                starts.append(row)
            for e in range(self.experts_per_rank):
                for src in range(self.ep_size):
                    n = recv_mat[src][e]
                    if n:
                        order.append(torch.arange(starts[src][e], starts[src][e] + n, device=x.device))
            perm = torch.cat(order) if order else torch.zeros(0, dtype=torch.long, device=x.device)
            local_sizes = [sum(recv_mat[src][e] for src in range(self.ep_size)) for e in range(self.experts_per_rank)]
            y = self.mlp(got.index_select(0, perm), local_sizes)
            back = torch.empty_like(y)
            back = back.index_copy(0, perm, y)
            out_sorted = _AllToAllRows.apply(back, recv_sizes, send_sizes, group)
        else:
            out_sorted = self.mlp(routed, tpe)
        w_sorted = expert_weights.reshape(-1).index_select(0, indices).to(out_sorted.dtype)
        out = torch.zeros_like(x2)
        out = out.index_add(0, token_of_copy, out_sorted * w_sorted.unsqueeze(-1))
        return out.view(in_shape)


class ParallelDroplessMoE(nn.Module):
    def __init__(self, neox_args, init_method, output_layer_init_method):
        super().__init__()
        if neox_args.moe_router_type == "sinkhorn":
            self.router = SinkhornRouter(neox_args, init_method)
        elif neox_args.moe_router_type == "topk":
            self.router = TopKTokenChoiceRouter(neox_args, init_method)
        else:
            raise ValueError(f"Invalid MoE Router type {neox_args.moe_router_type}")
        self.experts = ParallelDroplessMLP(neox_args, init_method=init_method,
                                           output_layer_init_method=output_layer_init_method)
        self.sequence_parallel = bool(neox_args.sequence_parallel) and mpu.get_model_parallel_world_size() > 1

    def forward(self, x):
        expert_weights, expert_indices = self.router(x)
        return self.experts(x, expert_weights, expert_indices)
