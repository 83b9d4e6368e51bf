"""RWKV-6 ("Finch") residual layer: data-dependent token shift, WKV recurrence, channel mix
(megatron/model/rwkv/v6/rwkv.py:100-366).

Differences from the reference, both deliberate:
* activations are ``[seq, batch, hidden]`` like the rest of the stack, and *time is the sequence
  dimension*: the token shift and the recurrence run along dim 0.  (The reference unpacks that tensor as
  ``B, T, C = x.size()`` and therefore shifts and recurs along the batch dimension, rwkv.py:188-191,221.)
* the WKV kernel (csrc/wkv6.cu) takes the sequence length at run time and works on strided views, so no
  per-sequence-length JIT build (rwkv.py:322-339) and no ``.contiguous()`` copies.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.gemm import linear
from ..ops.norm import layer_norm
from ..ops.wkv import wkv6


def _dev_dtype(neox_args):
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and \
        not neox_args.use_cpu_initialization else torch.device("cpu")
    return dev, neox_args.params_dtype


def _time_shift(x):
    """x [t, b, c] -> x_{t-1} (zeros at t = 0)."""
    return F.pad(x, (0, 0, 0, 0, 1, 0))[:-1]


def _position_ramp(hidden):
    return (torch.arange(hidden, dtype=torch.float32) / hidden).view(1, 1, hidden)


class _Lin(nn.Module):
    """Bias-free projection on the tcgen05 GEMM (nn.Linear parameter naming: ``weight`` [out, in])."""

    def __init__(self, n_in, n_out, dev, dt):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_out, n_in, device=dev, dtype=dt))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def forward(self, x):
        return linear(x, self.weight, None)


class RWKV_TimeMix(nn.Module):
    def __init__(self, neox_args, layer_number):
        super().__init__()
        self.neox_args, self.layer_number = neox_args, layer_number
        h, da, L = neox_args.hidden_size, neox_args.dim_att, neox_args.num_layers
        dev, dt = _dev_dtype(neox_args)
        r01 = layer_number / max(L - 1, 1)
        r10 = 1.0 - layer_number / L
        ddd = _position_ramp(h)
        mk = lambda t: nn.Parameter(t.to(device=dev, dtype=dt))
        self.time_maa_x = mk(1.0 - ddd.pow(r10))
        self.time_maa_w = mk(1.0 - ddd.pow(r10))
        self.time_maa_k = mk(1.0 - ddd.pow(r10))
        self.time_maa_v = mk(1.0 - (ddd.pow(r10) + 0.3 * r01))
        self.time_maa_r = mk(1.0 - ddd.pow(0.5 * r10))
        self.time_maa_g = mk(1.0 - ddd.pow(0.5 * r10))
        mix_dim, decay_dim = 32, 64
        self.time_maa_w1 = mk(torch.zeros(h, mix_dim * 5).uniform_(-1e-4, 1e-4))
        self.time_maa_w2 = mk(torch.zeros(5, mix_dim, h).uniform_(-1e-4, 1e-4))
        n = torch.arange(da, dtype=torch.float32)
        self.time_decay = mk((-6 + 5 * (n / max(da - 1, 1)) ** (0.7 + 1.3 * r01)).view(1, 1, da))
        self.time_decay_w1 = mk(torch.zeros(h, decay_dim).uniform_(-1e-4, 1e-4))
        self.time_decay_w2 = mk(torch.zeros(decay_dim, da).uniform_(-1e-4, 1e-4))
        zigzag = ((n + 1) % 3 - 1) * 0.1
        self.time_faaaa = mk((r01 * (1 - n / max(da - 1, 1)) + zigzag).view(neox_args.num_attention_heads,
                                                                           neox_args.head_size))
        self.receptance = _Lin(h, da, dev, dt)
        self.key = _Lin(h, da, dev, dt)
        self.value = _Lin(h, da, dev, dt)
        self.output = _Lin(da, h, dev, dt)
        self.gate = _Lin(h, da, dev, dt)
        self.ln_x = nn.GroupNorm(neox_args.num_attention_heads, da, eps=1e-5 * 64, device=dev, dtype=dt)

    def projections(self, x):
        """x [t, b, h] -> r, k, v, g, w, all [t, b, dim_att]."""
        T, B, C = x.shape
        xx = _time_shift(x) - x
        xxx = x + xx * self.time_maa_x
        xxx = torch.tanh(xxx.reshape(T * B, C) @ self.time_maa_w1).view(T * B, 5, -1).transpose(0, 1)
        mw, mk, mv, mr, mg = torch.bmm(xxx, self.time_maa_w2).view(5, T, B, C).unbind(0)
        xw = x + xx * (self.time_maa_w + mw)
        xk = x + xx * (self.time_maa_k + mk)
        xv = x + xx * (self.time_maa_v + mv)
        xr = x + xx * (self.time_maa_r + mr)
        xg = x + xx * (self.time_maa_g + mg)
        r, k, v = self.receptance(xr), self.key(xk), self.value(xv)
        g = F.silu(self.gate(xg))
        w = self.time_decay + torch.tanh(xw @ self.time_decay_w1) @ self.time_decay_w2
        return r, k, v, g, w

    def forward(self, x):
        T, B, C = x.shape
        r, k, v, g, w = self.projections(x)
        tb = lambda t: t.transpose(0, 1)                                  # [b, t, c] views of time-major data
        y = tb(wkv6(tb(r), tb(k), tb(v), tb(w.to(r.dtype)), self.time_faaaa))
        da = y.shape[-1]
        y = self.ln_x(y.reshape(T * B, da)).view(T, B, da)
        return self.output(y * g)


class RWKV_ChannelMix(nn.Module):
    def __init__(self, neox_args, layer_number):
        super().__init__()
        self.neox_args, self.layer_number = neox_args, layer_number
        h = neox_args.hidden_size
        dev, dt = _dev_dtype(neox_args)
        r10 = 1.0 - layer_number / neox_args.num_layers
        ddd = _position_ramp(h)
        self.time_maa_k = nn.Parameter((1.0 - ddd.pow(r10)).to(device=dev, dtype=dt))
        self.time_maa_r = nn.Parameter((1.0 - ddd.pow(r10)).to(device=dev, dtype=dt))
        self.key = _Lin(h, neox_args.ffn_dim, dev, dt)
        self.receptance = _Lin(h, h, dev, dt)
        self.value = _Lin(neox_args.ffn_dim, h, dev, dt)

    def forward(self, x):
        xx = _time_shift(x) - x
        xk = x + xx * self.time_maa_k
        xr = x + xx * self.time_maa_r
        k = torch.relu(self.key(xk)) ** 2
        return torch.sigmoid(self.receptance(xr)) * self.value(k)


class _LN(nn.Module):
    def __init__(self, h, dev, dt):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(h, device=dev, dtype=dt))
        self.bias = nn.Parameter(torch.zeros(h, device=dev, dtype=dt))

    def forward(self, x):
        return layer_norm(x, self.weight, self.bias, 1e-5)


class RWKVResidualLayer(nn.Module):
    def __init__(self, neox_args, layer_number):
        super().__init__()
        self.neox_args, self.layer_number = neox_args, layer_number
        assert neox_args.intermediate_size is None or neox_args.expansion_factor is None, \
            "Must pass either the absolute intermediate size or the relative expansion factor"
        if not getattr(neox_args, "dim_att", None):
            neox_args.dim_att = neox_args.hidden_size
        if neox_args.intermediate_size:
            ffn = neox_args.intermediate_size
        else:
            ffn = int((neox_args.expansion_factor or 3.5) * neox_args.hidden_size)
        neox_args.ffn_dim = int(ffn // 32 * 32)
        assert neox_args.hidden_size % 32 == 0 and neox_args.dim_att % 32 == 0 and neox_args.ffn_dim % 32 == 0
        assert neox_args.dim_att % neox_args.num_attention_heads == 0
        neox_args.head_size = neox_args.dim_att // neox_args.num_attention_heads
        self.head_size, self.num_attention_heads = neox_args.head_size, neox_args.num_attention_heads
        dev, dt = _dev_dtype(neox_args)
        self.ln1 = _LN(neox_args.hidden_size, dev, dt)
        self.ln2 = _LN(neox_args.hidden_size, dev, dt)
        self.att = RWKV_TimeMix(neox_args, layer_number)
        self.ffn = RWKV_ChannelMix(neox_args, layer_number)
        self.drop0 = nn.Dropout(neox_args.attention_dropout) if neox_args.attention_dropout > 0 else None
        self.drop1 = nn.Dropout(neox_args.hidden_dropout) if neox_args.hidden_dropout > 0 else None

    def forward(self, x):
        if self.layer_number == 0:
            x = self.ln1(x)
        x = x + self.att(self.ln1(x))
        if self.drop0 is not None:
            x = self.drop0(x)
        x = x + self.ffn(self.ln2(x))
        if self.drop1 is not None:
            x = self.drop1(x)
        return x


class RWKVResidualLayerPipe(RWKVResidualLayer):
    def forward(self, args):
        assert len(args) == 2
        hidden_states, mask = args
        return super().forward(hidden_states), mask


def RUN_CUDA_RWKV(B, T, C, H, r, k, v, w, u):
    """The WKV-6 recurrence under the reference's entry point (megatron/model/rwkv/v6/rwkv.py:95): ``r k v w``
    are ``[B, T, C]``, ``u`` is ``[H, C // H]``; any ``T`` (no compile-time sequence length)."""
    from ..ops.wkv import wkv6
    assert r.shape == (B, T, C) and u.shape[0] == H
    return wkv6(r, k, v, w, u)
