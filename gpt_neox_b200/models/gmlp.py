"""gMLP / aMLP block (megatron/model/gmlp.py:28-141): column-parallel up-projection, activation, causal
spatial gating unit (optionally with a one-head "tiny attention"), row-parallel down-projection.

The spatial projection keeps the ``[seq, batch, channel]`` layout: for a fixed (batch, channel) pair the
gate is ``tril(W) @ gate``, i.e. one GEMM ``tril(W)[s, s] @ gate[s, (b d)]`` on the tcgen05 kernel with the
activation as the K-major operand, where the reference transposes to ``[b, d, s]`` and back
(gmlp.py:69-85).  The tiny attention runs on the flash-attention kernel with one head.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import parallel as mpu
from ..ops.attention import attention_reference, flash_attention
from ..ops.gemm import gemm, linear
from .activations import get_activation
from .norms import get_norm


def _dev_dtype(neox_args):
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and \
        not neox_args.use_cpu_initialization else torch.device("cpu")
    return dev, neox_args.params_dtype


class _SpatialProj(torch.autograd.Function):
    """out[s, n] = W[s, s] @ g[s, n] on the tcgen05 GEMM (W already masked)."""

    @staticmethod
    def forward(ctx, w, g):
        ctx.save_for_backward(w, g)
        return gemm(w, g, trans_b=True)

    @staticmethod
    def backward(ctx, go):
        w, g = ctx.saved_tensors
        go = go.contiguous()
        gg = gemm(w, go, trans_a=True, trans_b=True)           # W^T go
        gw = gemm(go, g)                                        # go g^T : g is [s, n] = "[N_out, K]"
        return gw, gg


class TinyAttention(nn.Module):
    def __init__(self, neox_args, d_attn, d_ff, mask_fn):
        super().__init__()
        dev, dt = _dev_dtype(neox_args)
        self.proj_qkv = nn.Linear(d_ff * 2, 3 * d_attn, device=dev, dtype=dt)
        self.scale = d_attn ** -0.5
        self.d_attn = d_attn
        self.proj_ffn = nn.Linear(d_attn, d_ff, device=dev, dtype=dt)

    def forward(self, x, attention_mask):
        """x [s, b, 2 d_ff] -> [s, b, d_ff]; causal, one head."""
        s, b, _ = x.shape
        qkv = linear(x, self.proj_qkv.weight, self.proj_qkv.bias)
        q, k, v = (t.transpose(0, 1).unsqueeze(2) for t in qkv.chunk(3, dim=-1))      # [b, s, 1, d]
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and self.d_attn in (64, 128):
            o = flash_attention(q.contiguous(), k.contiguous(), v.contiguous(), scale=self.scale, causal=True)
        else:
            o, _ = attention_reference(q, k, v, scale=self.scale, causal=True)
        o = o.squeeze(2).transpose(0, 1)
        return linear(o.contiguous(), self.proj_ffn.weight, self.proj_ffn.bias)


class SpatialGatingUnit(nn.Module):
    def __init__(self, neox_args, d_ff, d_attn=None, causal=True, mask_fn=None):
        super().__init__()
        self.causal = causal
        self.use_attn = d_attn is not None
        norm, eps = get_norm(neox_args)
        self.norm = norm(d_ff, eps=eps)
        dev, dt = _dev_dtype(neox_args)
        self.proj = nn.Linear(neox_args.seq_length, neox_args.seq_length, device=dev, dtype=dt)
        if self.use_attn:
            assert mask_fn is not None
            self.attn = TinyAttention(neox_args=neox_args, d_attn=d_attn, d_ff=d_ff, mask_fn=mask_fn)
        nn.init.zeros_(self.proj.weight)
        nn.init.constant_(self.proj.bias, 1.0)

    def forward(self, x, attention_mask):
        """x [s, b, 2 d] -> [s, b, d]."""
        n, b, _ = x.shape
        res, gate = x.chunk(2, dim=-1)
        gate = self.norm(gate.contiguous())
        weight, bias = self.proj.weight[:n, :n], self.proj.bias[:n]
        if self.causal:
            weight = torch.tril(weight)
        d = gate.shape[-1]
        g2 = gate.reshape(n, b * d)
        if g2.is_cuda and g2.dtype in (torch.bfloat16, torch.float16) and n % 8 == 0 and (b * d) % 8 == 0:
            out = _SpatialProj.apply(weight.contiguous(), g2)
        else:
            out = weight @ g2
        gate = out.view(n, b, d) + bias.view(n, 1, 1)
        if self.use_attn:
            gate = gate + self.attn(x, attention_mask)
        return gate * res


class GMLPBlock(nn.Module):
    def __init__(self, neox_args, init_method, output_layer_init_method, layer_number, ff_mult=4, mask_fn=None):
        super().__init__()
        self.layer_number = layer_number
        ff_dim = neox_args.hidden_size * ff_mult
        norm, eps = get_norm(neox_args)
        self.norm = norm(neox_args.hidden_size, eps=eps)
        self.input_linear = mpu.ColumnParallelLinear(neox_args=neox_args, input_size=neox_args.hidden_size,
                                                     output_size=ff_dim * 2, gather_output=False,
                                                     init_method=init_method, skip_bias_add=True)
        self.activation_func, _ = get_activation(neox_args)
        ff_dim_parallel = mpu.divide(ff_dim, mpu.get_model_parallel_world_size())
        d_attn = neox_args.gmlp_attn_dim if neox_args.attention_config[layer_number] == "amlp" else None
        self.sgu = SpatialGatingUnit(neox_args, ff_dim_parallel, d_attn, causal=True, mask_fn=mask_fn)
        self.output_linear = mpu.RowParallelLinear(neox_args=neox_args, input_size=ff_dim,
                                                   output_size=neox_args.hidden_size, input_is_parallel=True,
                                                   init_method=output_layer_init_method, skip_bias_add=True)

    def forward(self, args):
        assert len(args) == 2, "GMLPBlock expects 2 arguments"
        x, attention_mask = args
        x = self.norm(x)
        x, _ = self.input_linear(x)
        x = self.activation_func(x)
        x = self.sgu(x, attention_mask)
        x, _ = self.output_linear(x)
        return x, attention_mask
