"""Block-level fused operators built from the kernels of this library.

* ``mlp_gelu``     linear1 -> bias + GeLU -> linear2 (+ bias + residual) as ONE autograd node:
                   GeLU and its derivative live in GEMM epilogues, so neither forward nor backward
                   launches an element-wise kernel (the reference fuses only bias+GeLU through
                   torch.jit, megatron/model/activations.py:78-112).
* ``qkv_attention``  rotary (partial, in place on the fused QKV projection output) + causal flash
                   attention reading q / k / v as strided views of that buffer + gradients written
                   back into one buffer of the same layout: no de-interleave, transpose or
                   concatenation copies (the reference does view/split/permute/contiguous around
                   flash-attn, megatron/model/transformer.py:800-894).
CPU tensors take the PyTorch statement of the same math.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib
from .attention import _fwd as _attn_fwd_launch
from .attention import _strides_bhs, attention_reference
from .elementwise import bias_grad, colsum
from .gemm import LAUNCHES, gemm, wgrad
from .rope import _launch as _rope_launch
from .rope import apply_rotary


class _MLPGeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, kind, recompute_act):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        # aux: the pre-activation when the activation is recomputed in backward, otherwise gelu'(pre-activation)
        # so that the backward GEMM epilogue is one multiply
        pre = torch.empty((M, w1.shape[0]), device=x.device, dtype=x.dtype)
        h = gemm(x2, w1, bias=b1, gelu=kind, aux_out=pre, aux_deriv=not recompute_act)
        r2 = residual.reshape(M, -1) if residual is not None else None
        if r2 is not None and not r2.is_contiguous():
            r2 = r2.contiguous()
        y = gemm(h, w2, bias=b2, residual=r2)
        ctx.kind, ctx.recompute_act = kind, recompute_act
        ctx.has_b1, ctx.has_b2, ctx.has_res = b1 is not None, b2 is not None, residual is not None
        ctx.x_shape = x.shape
        ctx.biases = (b1, b2)           # the parameters themselves: their main_grad takes the bias gradients
        ctx.save_for_backward(x2, w1, b1, w2, pre, None if recompute_act else h)
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w1, b1, w2, pre, h = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        if h is None:
            from .elementwise import bias_act
            h = bias_act(pre, None, "gelu_tanh" if ctx.kind == "tanh" else "gelu")
        # d(pre) = (gy @ W2) * gelu'(pre)   -- derivative applied in the GEMM epilogue
        dpre = gemm(gy2, w2, trans_b=True, dgelu_aux=pre, dgelu=ctx.kind if ctx.recompute_act else "mul")
        gw2 = wgrad(gy2, h, w2) if ctx.needs_input_grad[3] else None
        gb2 = bias_grad(gy2, ctx.biases[1]) if (ctx.has_b2 and ctx.needs_input_grad[4]) else None
        gx = gemm(dpre, w1, trans_b=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        gw1 = wgrad(dpre, x2, w1) if ctx.needs_input_grad[1] else None
        gb1 = bias_grad(dpre, ctx.biases[0]) if (ctx.has_b1 and ctx.needs_input_grad[2]) else None
        gres = gy2.view(gy.shape) if ctx.has_res else None     # contiguous from here on down the stack
        return gx, gw1, gb1, gw2, gb2, gres, None, None


def mlp_gelu(x, w1, b1, w2, b2=None, residual=None, kind: str = "erf", recompute_act: bool = False):
    """``gelu(x @ w1^T + b1) @ w2^T (+ b2) (+ residual)``; kind in {"erf", "tanh"}."""
    if x.is_cuda and x.dtype in _lib.H16:
        return _MLPGeluFn.apply(x, w1, b1, w2, b2, residual, kind, recompute_act)
    if x.is_cuda:
        raise _lib.KernelError("mlp_gelu: CUDA path needs bf16")
    h = F.gelu(F.linear(x, w1, b1), approximate="tanh" if kind == "tanh" else "none")
    y = F.linear(h, w2, b2)
    return y if residual is None else y + residual


def _qkv_views(qkv, np_, kvp, hn):
    """q [s,b,np,hn], k / v [s,b,kvp,hn] strided views of the projection output [s,b,*]."""
    s, b = qkv.shape[0], qkv.shape[1]
    if kvp == np_:  # per-head interleaved [q_i, k_i, v_i]  (megatron/model/transformer.py:800-809)
        t = qkv.view(s, b, np_, 3 * hn)
        return t[..., :hn], t[..., hn:2 * hn], t[..., 2 * hn:]
    # grouped-query layout [all q heads | all k heads | all v heads]  (transformer.py:725-740)
    q = qkv[..., : np_ * hn].view(s, b, np_, hn)
    k = qkv[..., np_ * hn:(np_ + kvp) * hn].view(s, b, kvp, hn)
    v = qkv[..., (np_ + kvp) * hn:].view(s, b, kvp, hn)
    return q, k, v


class _QKVAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, np_, kvp, hn, rot, pos0, scale, window, alibi, dropout_p=0.0, seed=0):
        s, b = qkv.shape[0], qkv.shape[1]
        q, k, v = _qkv_views(qkv, np_, kvp, hn)
        if rot > 0:
            _rope_launch(q, q, cos, sin, rot, pos0, False)
            _rope_launch(k, k, cos, sin, rot, pos0, False)
        qb, kb, vb = (t.permute(1, 0, 2, 3) for t in (q, k, v))  # [b, s, heads, hn] views
        out = torch.empty((s, b, np_, hn), device=qkv.device, dtype=qkv.dtype)
        ob = out.permute(1, 0, 2, 3)
        sq_pad = (s + 127) // 128 * 128
        lse = torch.full((b, np_, sq_pad), float("inf"), device=qkv.device, dtype=torch.float32)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(qkv).nx_flash_attn_fwd(
            _lib.ptr(qb), _lib.ptr(kb), _lib.ptr(vb), _lib.ptr(ob), _lib.ptr(lse), _lib.ptr(alibi),
            b, np_, kvp, s, s, hn, *_strides_bhs(qb), *_strides_bhs(kb), *_strides_bhs(vb), *_strides_bhs(ob),
            float(scale), 1, int(window), float(dropout_p), int(seed), None, None, 0, _lib.stream()),
            "nx_flash_attn_fwd")
        ctx.save_for_backward(qkv, out, lse, cos, sin, alibi)
        ctx.cfg = (np_, kvp, hn, rot, pos0, scale, window)
        ctx.dropout = (float(dropout_p), int(seed))
        return out.view(s, b, np_ * hn)

    @staticmethod
    def backward(ctx, gout):
        qkv, out, lse, cos, sin, alibi = ctx.saved_tensors
        np_, kvp, hn, rot, pos0, scale, window = ctx.cfg
        s, b = qkv.shape[0], qkv.shape[1]
        if not gout.is_contiguous():
            gout = gout.contiguous()
        q, k, v = _qkv_views(qkv, np_, kvp, hn)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _qkv_views(dqkv, np_, kvp, hn)
        perm = lambda t: t.permute(1, 0, 2, 3)
        qb, kb, vb, dqb, dkb, dvb = map(perm, (q, k, v, dq, dk, dv))
        ob = perm(out)
        dob = perm(gout.view(s, b, np_, hn))
        # (rows beyond the sequence exist only when it is not a multiple of the 128-row tile: only then a fill)
        delta = (torch.empty if lse.shape[-1] == s else torch.zeros)(lse.shape, device=qkv.device, dtype=torch.float32)
        LAUNCHES["n"] += 3
        _lib.check(_lib.lib(qkv).nx_flash_attn_bwd(
            _lib.ptr(qb), _lib.ptr(kb), _lib.ptr(vb), _lib.ptr(ob), _lib.ptr(dob), _lib.ptr(lse),
            _lib.ptr(delta), _lib.ptr(dqb), _lib.ptr(dkb), _lib.ptr(dvb), _lib.ptr(alibi),
            b, np_, kvp, s, s, hn, *_strides_bhs(qb), *_strides_bhs(kb), *_strides_bhs(vb), *_strides_bhs(ob),
            *_strides_bhs(dob), *_strides_bhs(dqb), *_strides_bhs(dkb), *_strides_bhs(dvb),
            float(scale), 1, int(window), ctx.dropout[0], ctx.dropout[1], None, None, 0, _lib.stream()),
            "nx_flash_attn_bwd")
        if rot > 0:
            _rope_launch(dq, dq, cos, sin, rot, pos0, True)
            _rope_launch(dk, dk, cos, sin, rot, pos0, True)
        return (dqkv,) + (None,) * 12


def qkv_attention(qkv, *, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int = 0,
                  cos=None, sin=None, pos0: int = 0, scale: float | None = None, window: int = -1,
                  alibi=None, dropout_p: float = 0.0, seed: int | None = None):
    """Causal self-attention straight from the fused QKV projection output ``qkv`` [s, b, *]
    (heads are this rank's).  Returns the context [s, b, num_heads * head_dim]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    window = -1 if window is None else int(window)
    if dropout_p > 0 and seed is None:
        from .attention import next_dropout_seed
        seed = next_dropout_seed()
    seed = seed or 0
    if qkv.is_cuda:
        if qkv.dtype not in _lib.H16 or head_dim % 8 or head_dim > 128:
            raise _lib.KernelError(f"qkv_attention: CUDA path needs bf16 and head dim % 8 == 0, <= 128 "
                                   f"(got {qkv.dtype}, {head_dim})")
        if not qkv.is_contiguous():
            qkv = qkv.contiguous()
        if alibi is not None:
            alibi = alibi.to(device=qkv.device, dtype=torch.float32).contiguous()
        return _QKVAttentionFn.apply(qkv, cos, sin, num_heads, num_kv_heads, head_dim, rotary_dim, pos0,
                                     scale, window, alibi, float(dropout_p), seed)
    s, b = qkv.shape[0], qkv.shape[1]
    q, k, v = _qkv_views(qkv, num_heads, num_kv_heads, head_dim)
    if rotary_dim > 0:
        q = apply_rotary(q, cos, sin, rotary_dim, pos0)
        k = apply_rotary(k, cos, sin, rotary_dim, pos0)
    o, _ = attention_reference(q.permute(1, 0, 2, 3), k.permute(1, 0, 2, 3), v.permute(1, 0, 2, 3),
                               scale=scale, causal=True, window=window, alibi=alibi, dropout_p=dropout_p, seed=seed)
    return o.permute(1, 0, 2, 3).reshape(s, b, num_heads * head_dim)
