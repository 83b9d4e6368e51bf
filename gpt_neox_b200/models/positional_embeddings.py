"""Positional embeddings: rotary tables, sinusoidal, ALiBi
(megatron/model/positional_embeddings.py:19-257)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops.attention import alibi_slopes
from ..ops.rope import rotary_tables


class SinusoidalPositionalEmbedding(nn.Module):
    def __init__(self, dim, base=10000, precision=torch.half):
        super().__init__()
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.precision = precision

    def forward(self, x, seq_dim=1):
        """``x``: an integer tensor of position ids [b, s] -> the table rows of those positions [b, s, dim] (so a
        decoding step with a KV cache, which feeds one token at position t, gets row t and not row 0); any other
        tensor -> rows 0 .. s-1 along ``seq_dim`` as [1, s, dim]."""
        if not x.is_floating_point() and x.dim() == 2:
            sinusoid_inp = x.to(self.inv_freq.dtype).unsqueeze(-1) * self.inv_freq
            if self.precision == torch.bfloat16:
                sinusoid_inp = sinusoid_inp.float()
            sin, cos = sinusoid_inp.sin(), sinusoid_inp.cos()
            if self.precision == torch.bfloat16:
                sin, cos = sin.bfloat16(), cos.bfloat16()
            return torch.cat((sin, cos), dim=-1)
        t = torch.arange(x.shape[seq_dim], device=x.device).type_as(self.inv_freq)
        sinusoid_inp = torch.einsum("i,j->ij", t, self.inv_freq)
        if self.precision == torch.bfloat16:
            sinusoid_inp = sinusoid_inp.float()
        sin, cos = sinusoid_inp.sin(), sinusoid_inp.cos()
        if self.precision == torch.bfloat16:
            sin, cos = sin.bfloat16(), cos.bfloat16()
        emb = torch.cat((sin, cos), dim=-1)
        return emb[None, :, :]


class RotaryEmbedding(nn.Module):
    """Holds fp32 cos / sin tables [max_seq_len, dim/2] (``emb = cat(freqs, freqs)`` of the reference
    duplicates the halves; the kernels index the half table twice instead)."""

    def __init__(self, dim, max_seq_len, base=10000, precision=torch.half, save_inv_freqs=False):
        super().__init__()
        self.dim, self.base, self.max_seq_len, self.precision = dim, base, max_seq_len, precision
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=save_inv_freqs)
        cos, sin = rotary_tables(dim, max_seq_len, base)
        self.register_buffer("cos_table", cos, persistent=False)
        self.register_buffer("sin_table", sin, persistent=False)

    def forward(self, x=None, seq_dim=0, seq_len=None):
        """(cos, sin) tables; asserts the requested length fits the precomputed range."""
        if seq_len is None and x is not None:
            seq_len = x.shape[seq_dim]
        assert seq_len is None or seq_len <= self.max_seq_len
        return self.cos_table, self.sin_table


class AliBi(nn.Module):
    """ALiBi slopes for this tensor-parallel rank's heads; ``forward`` adds the dense bias
    ``-slope * (i - j)`` to attention scores [b, np, sq, sk] (non-flash path); the flash path takes
    ``self.slopes`` directly."""

    def __init__(self, num_heads, mp_size=1, mp_rank=0):
        super().__init__()
        assert mp_size <= num_heads and mp_rank <= mp_size
        self.mp_size, self.mp_rank, self.num_heads = mp_size, mp_rank, num_heads
        self.slice_size = num_heads // mp_size
        slopes = alibi_slopes(num_heads)[mp_rank * self.slice_size:(mp_rank + 1) * self.slice_size]
        self.register_buffer("slopes", slopes.contiguous(), persistent=False)

    def bias(self, seq_len_q, seq_len_k, device, dtype):
        qpos = torch.arange(seq_len_q, device=device)[:, None] + (seq_len_k - seq_len_q)
        kpos = torch.arange(seq_len_k, device=device)[None, :]
        rel = (kpos - qpos).clamp(max=0).to(torch.float32)
        return (self.slopes.to(device)[:, None, None] * rel[None]).to(dtype)

    def forward(self, x):
        sq, sk = x.shape[-2], x.shape[-1]
        return x + self.bias(sq, sk, x.device, x.dtype)[None]


# ------------------------------------------------------------------ functional rotary helpers
def rotate_half(x):
    """``[x1 | x2] -> [-x2 | x1]`` on the last dimension."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary_pos_emb_torch(q, k, cos, sin, offset: int = 0):
    """Rotate ``q`` and ``k`` (``[s, b, heads, d]``) with tables ``[>= offset + s, 1, 1, d]`` whose two halves
    are equal (megatron/model/positional_embeddings.py apply_rotary_pos_emb*).  Plain PyTorch in the
    tables' precision; the model itself uses the kernel in `ops.rope`."""
    s = q.shape[0]
    c, sn = cos[offset:offset + s], sin[offset:offset + s]
    return (q * c) + (rotate_half(q) * sn), (k * c) + (rotate_half(k) * sn)


apply_rotary_pos_emb = apply_rotary_pos_emb_torch
