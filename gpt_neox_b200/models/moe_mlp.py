"""Expert MLPs over variable-size row groups (megatron/model/moe_mlp.py:134-451): one weight tensor
holds all local experts, ``[experts_local * ffn, h]``; rows of the input are grouped by expert and
``tokens_per_expert`` gives the group sizes.  The grouped matmul runs the tcgen05 GEMM once per
non-empty expert on row slices of the grouped activations (csrc/gemm_tcgen05.cu)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import parallel as mpu
from ..ops.gemm import linear
from .activations import get_activation


class ScaleGradient(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad * ctx.scale, None


scale_gradient = ScaleGradient.apply


def _device(neox_args):
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and \
        not getattr(neox_args, "use_cpu_initialization", False) else torch.device("cpu")


def _init_expert_weight(param, init_fn, neox_args, num_experts):
    """Every expert gets its own draw whatever the expert-parallel size: under host initialisation the
    full ``[experts * ffn, h]`` matrix is drawn and this rank's experts sliced out (identical weights for
    every expert-parallel layout); on the device each expert-parallel rank draws from its own stream."""
    ep = mpu.get_expert_parallel_world_size()
    if ep == 1:
        init_fn(param)
        return
    r = mpu.get_expert_parallel_rank()
    if getattr(neox_args, "use_cpu_initialization", False):
        master = torch.empty(param.shape[0] * ep, param.shape[1], dtype=torch.float32)
        init_fn(master)
        with torch.no_grad():
            param.copy_(master[r * param.shape[0]:(r + 1) * param.shape[0]])
        return
    devs = [param.device] if param.is_cuda else []
    with torch.random.fork_rng(devices=devs):
        torch.manual_seed(torch.initial_seed() + 7919 * (r + 1))
        init_fn(param)


def grouped_linear(x, w, sizes, trans_b: bool):
    """Row group e of ``x`` times expert e's matrix. ``w``: [E, ffn, h]; trans_b: x @ w[e]^T (h -> ffn),
    else x @ w[e] (ffn -> h). ``sizes``: python list of group sizes."""
    outs, start = [], 0
    for e, n in enumerate(sizes):
        if n == 0:
            continue
        xe = x[start:start + n]
        outs.append(linear(xe, w[e], None) if trans_b else _linear_nn(xe, w[e]))
        start += n
    if not outs:
        return x.new_zeros((0, w.shape[1] if trans_b else w.shape[2]))
    return torch.cat(outs, dim=0)


class _LinearNN(torch.autograd.Function):
    """y = x @ W with W [K, N] row-major (the second expert matrix is stored [ffn, h])."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops.gemm import gemm
        x = x.contiguous()
        ctx.save_for_backward(x, w)
        return gemm(x, w, trans_b=True)

    @staticmethod
    def backward(ctx, gy):
        from ..ops.gemm import gemm
        x, w = ctx.saved_tensors
        gy = gy.contiguous()
        gx = gemm(gy, w)                                   # gy [M,N] @ W^T : W is [K,N] = "[N_out=K, K_red=N]"
        gw = gemm(x, gy, trans_a=True, trans_b=True)       # x^T gy : [K, N]
        return gx, gw


def _linear_nn(x, w):
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16):
        return _LinearNN.apply(x, w)
    return x @ w


class ParallelGroupedMLP(nn.Module):
    def __init__(self, neox_args, init_method, output_layer_init_method, stride=1, multiple_of=256):
        super().__init__()
        self.activation_func, self.activation_fn_is_gated = get_activation(neox_args)
        self.activation_type = neox_args.activation
        self.num_experts = neox_args.moe_num_experts
        ep = mpu.get_expert_parallel_world_size()
        self.experts_per_rank = self.num_experts // ep
        self.hidden_size = neox_args.hidden_size
        if neox_args.intermediate_size is not None:
            ff = neox_args.intermediate_size
        else:
            ff = 4 * self.hidden_size
            ff = multiple_of * ((ff + multiple_of - 1) // multiple_of)
        self.per_expert_ff_dim = ff
        rows = self.experts_per_rank * ff
        dev, dt = _device(neox_args), neox_args.params_dtype
        self.w1 = nn.Parameter(torch.empty(rows, self.hidden_size, device=dev, dtype=dt))
        self.w2 = nn.Parameter(torch.empty(rows, self.hidden_size, device=dev, dtype=dt))
        _init_expert_weight(self.w1, init_method, neox_args, self.num_experts)
        _init_expert_weight(self.w2, output_layer_init_method, neox_args, self.num_experts)
        for p in (self.w1, self.w2):
            p.expert_parallel = ep > 1      # reduced over the expert-data-parallel group only

    def forward(self, x, tokens_per_expert):
        sizes = tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else list(tokens_per_expert)
        w1 = self.w1.view(self.experts_per_rank, -1, self.hidden_size)
        w2 = self.w2.view(self.experts_per_rank, -1, self.hidden_size)
        h = grouped_linear(x, w1, sizes, trans_b=True)
        h = self.activation_func(h)
        return grouped_linear(h, w2, sizes, trans_b=False)


class ParallelGroupedLLaMAMLP(nn.Module):
    """Gated expert MLP: ``w2(act(w1 x) * w3 x)`` per expert."""

    def __init__(self, neox_args, init_method, output_layer_init_method, stride=1, multiple_of=256):
        super().__init__()
        self.activation_func, _ = get_activation(neox_args)
        self.activation_type = neox_args.activation
        self.num_experts = neox_args.moe_num_experts
        ep = mpu.get_expert_parallel_world_size()
        self.experts_per_rank = self.num_experts // ep
        self.hidden_size = neox_args.hidden_size
        if neox_args.intermediate_size is not None:
            ff = neox_args.intermediate_size
        else:
            ff = int(2 * neox_args.hidden_size * 4 / 3)
            ff = multiple_of * ((ff + multiple_of - 1) // multiple_of)
        self.per_expert_ff_dim = ff
        rows = self.experts_per_rank * ff
        dev, dt = _device(neox_args), neox_args.params_dtype
        self.w1 = nn.Parameter(torch.empty(rows, self.hidden_size, device=dev, dtype=dt))
        self.w3 = nn.Parameter(torch.empty(rows, self.hidden_size, device=dev, dtype=dt))
        self.w2 = nn.Parameter(torch.empty(rows, self.hidden_size, device=dev, dtype=dt))
        _init_expert_weight(self.w1, init_method, neox_args, self.num_experts)
        _init_expert_weight(self.w3, init_method, neox_args, self.num_experts)
        _init_expert_weight(self.w2, output_layer_init_method, neox_args, self.num_experts)
        for p in (self.w1, self.w2, self.w3):
            p.expert_parallel = ep > 1

    def forward(self, x, tokens_per_expert):
        sizes = tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else list(tokens_per_expert)
        v = lambda w: w.view(self.experts_per_rank, -1, self.hidden_size)
        gate = grouped_linear(x, v(self.w1), sizes, trans_b=True)
        up = grouped_linear(x, v(self.w3), sizes, trans_b=True)
        h = torch.nn.functional.silu(gate) * up
        return grouped_linear(h, v(self.w2), sizes, trans_b=False)


# The reference's "memory optimized" variants recompute the activation in backward to save one
# [tokens, ffn] tensor; the grouped kernels here always keep only the pre-activation (as its derivative),
# so the plain classes already have that footprint.
MemoryOptimizedParallelGroupedMLP = ParallelGroupedMLP
MemoryOptimizedParallelGroupedLLaMAMLP = ParallelGroupedLLaMAMLP
