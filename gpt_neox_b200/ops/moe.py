"""Dropless MoE expert computation on the device: routing plan -> padded permutation -> grouped tcgen05
GEMMs -> weighted combine (csrc/moe.cu, csrc/gemm_tcgen05.cu grouped modes).

Nothing in the layer reads the routing result on the host: buffer sizes are the static worst case
(``tokens * k + experts * 127`` rows, rounded to 128) and the kernels skip the unused tail by consulting
device-side tables.  Reference path: megatron/model/moe.py:62-160 (megablocks sort / gather / scatter) and
megatron/model/moe_mlp.py:212-223 (grouped_gemm, which needs the per-expert batch sizes on the CPU).
"""
from __future__ import annotations

import torch

from . import _lib
from .gemm import EPI_ACCUM, EPI_GELU_ERF, EPI_GELU_TANH, EPI_OUT_F32, LAUNCHES, aux_flags


class Plan:
    """Device-side routing plan of one layer call."""

    def __init__(self, expert_indices: torch.Tensor, num_experts: int):
        L = _lib.lib()
        idx = expert_indices.reshape(-1).contiguous()
        if idx.dtype != torch.int64:
            idx = idx.long()
        self.C, self.E, self.k = idx.numel(), num_experts, expert_indices.shape[-1]
        dev = idx.device
        nblk = L.nx_moe_blocks(self.C)
        self.max_rows = L.nx_moe_max_rows(self.C, num_experts)
        i32 = lambda n: torch.empty(n, device=dev, dtype=torch.int32)
        hist, base = i32(nblk * num_experts), i32(nblk * num_experts)
        self.counts, self.offsets = i32(num_experts), i32(num_experts + 1)
        self.tile_expert = i32(self.max_rows // 128)
        self.dest_row, self.src_copy = i32(self.C), i32(self.max_rows)
        LAUNCHES["n"] += 3
        _lib.check(L.nx_moe_plan(_lib.ptr(idx), self.C, num_experts, _lib.ptr(hist), _lib.ptr(base),
                                 _lib.ptr(self.counts), _lib.ptr(self.offsets), _lib.ptr(self.tile_expert),
                                 _lib.ptr(self.dest_row), _lib.ptr(self.src_copy), _lib.stream()), "nx_moe_plan")


def gather_rows(src, plan: Plan, scale=None):
    """[T, H] -> padded permuted [max_rows, H]: row r = (scale[c] *) src[c // k] with c = src_copy[r], 0 for padding."""
    H = src.shape[1]
    out = torch.empty((plan.max_rows, H), device=src.device, dtype=src.dtype)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(src).nx_moe_gather_rows(_lib.ptr(src), src.stride(0), _lib.ptr(plan.src_copy), _lib.ptr(scale),
                                             plan.k, _lib.ptr(out), plan.max_rows, H, _lib.stream()),
               "nx_moe_gather_rows")
    return out


def combine(y, plan: Plan, weights=None):
    """padded permuted [max_rows, H] -> [T, H]: sum over the k copies of each token (weighted)."""
    T, H = plan.C // plan.k, y.shape[1]
    out = torch.empty((T, H), device=y.device, dtype=y.dtype)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(y).nx_moe_combine(_lib.ptr(y), _lib.ptr(plan.dest_row), _lib.ptr(weights), plan.k,
                                         _lib.ptr(out), T, H, _lib.stream()), "nx_moe_combine")
    return out


def weight_grad(g, y, plan: Plan):
    dw = torch.empty(plan.C, device=g.device, dtype=g.dtype)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(g).nx_moe_weight_grad(_lib.ptr(g), _lib.ptr(y), _lib.ptr(plan.dest_row), plan.k,
                                             _lib.ptr(dw), plan.C, g.shape[1], _lib.stream()), "nx_moe_weight_grad")
    return dw


def grouped_gemm_rows(a, w, plan: Plan, n_out, *, trans_b, gelu=None, aux_out=None, dgelu_aux=None, dgelu=None,
                      aux_deriv=False):
    """C[rows, n_out] = A[rows, K] x op(W_e) per 128-row tile; ``w`` stacks the experts' matrices
    ([E * n_out, K] for trans_b False, [E * K, n_out] for trans_b True)."""
    rows, K = a.shape
    out = torch.empty((rows, n_out), device=a.device, dtype=a.dtype)
    flags, ld_aux = 0, 0
    if gelu is not None:
        flags |= EPI_GELU_TANH if gelu == "tanh" else EPI_GELU_ERF
    flags |= aux_flags(gelu, aux_out, aux_deriv, dgelu_aux, dgelu)
    if aux_out is not None:
        ld_aux = aux_out.stride(0)
    if dgelu_aux is not None:
        ld_aux = dgelu_aux.stride(0)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(a).nx_gemm_bf16_grouped(1, _lib.ptr(a), _lib.ptr(w), _lib.ptr(out), rows, n_out, K, a.stride(0),
                                               w.stride(0), out.stride(0), int(trans_b), plan.E,
                                               _lib.ptr(plan.tile_expert), None, 0, _lib.ptr(dgelu_aux),
                                               _lib.ptr(aux_out), ld_aux, flags, _lib.stream()),
               "nx_gemm_bf16_grouped(rows)")
    return out


def grouped_wgrad(a, b, plan: Plan, weight):
    """dW_e [M, N] (+)= A[rows_e, M]^T B[rows_e, N] for every expert; accumulates into ``weight.main_grad``
    (fp32) when present, otherwise returns a new [E * M, N] tensor."""
    M, N = a.shape[1], b.shape[1]
    mg = getattr(weight, "main_grad", None)
    if mg is not None and mg.dtype == torch.float32:
        out, flags, ret = mg, EPI_ACCUM | EPI_OUT_F32, None
    else:
        out = torch.zeros((plan.E * M, N), device=a.device, dtype=a.dtype)
        flags, ret = 0, out
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(a).nx_gemm_bf16_grouped(2, _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, a.shape[0], a.stride(0),
                                               b.stride(0), N, 1, plan.E, None, _lib.ptr(plan.offsets), M * N, None,
                                               None, 0, flags, _lib.stream()), "nx_gemm_bf16_grouped(wgrad)")
    if ret is not None and mg is not None:
        mg.add_(ret.view_as(mg).to(mg.dtype))
        return None
    return ret


class _ExpertsGeluFn(torch.autograd.Function):
    """out[t] = sum_j w[t,j] * W2_e^T gelu(W1_e x_t), e = expert[t,j] — one autograd node for the layer."""

    @staticmethod
    def forward(ctx, x2, weights, indices, w1, w2, num_experts, kind):
        plan = Plan(indices, num_experts)
        ffn = w1.shape[0] // num_experts
        xp = gather_rows(x2, plan)
        pre = torch.empty((plan.max_rows, ffn), device=x2.device, dtype=x2.dtype)
        h = grouped_gemm_rows(xp, w1, plan, ffn, trans_b=False, gelu=kind, aux_out=pre, aux_deriv=True)  # gelu'(.)
        y = grouped_gemm_rows(h, w2, plan, w2.shape[1], trans_b=True)
        wf = weights.reshape(-1).contiguous()
        out = combine(y, plan, wf)
        ctx.save_for_backward(xp, pre, h, y, wf, w1, w2)
        ctx.plan, ctx.kind = plan, kind
        ctx.w_shape = weights.shape
        return out

    @staticmethod
    def backward(ctx, g):
        xp, pre, h, y, wf, w1, w2 = ctx.saved_tensors
        plan = ctx.plan
        g = g.contiguous()
        d_w = weight_grad(g, y, plan).view(ctx.w_shape)
        dy = gather_rows(g, plan, scale=wf)                               # [rows, hidden], zero padding
        dpre = grouped_gemm_rows(dy, w2, plan, w2.shape[0] // plan.E, trans_b=False, dgelu_aux=pre, dgelu="mul")
        dw2 = grouped_wgrad(h, dy, plan, w2)
        dxp = grouped_gemm_rows(dpre, w1, plan, w1.shape[1], trans_b=True)
        dw1 = grouped_wgrad(dpre, xp, plan, w1)
        dx = combine(dxp, plan, None)
        return dx, d_w, None, dw1, dw2, None, None


def experts_gelu(x2, weights, indices, w1, w2, num_experts, kind="erf"):
    """x2 [T, h] bf16; weights / indices [T, k]; w1, w2 [E * ffn, h]."""
    return _ExpertsGeluFn.apply(x2, weights.to(x2.dtype), indices, w1, w2, num_experts, kind)
