"""Causal flash attention (GQA, ALiBi, sliding window, dropout, cached decoding with sq != sk) on the tcgen05 kernels of
csrc/attention_fwd.cu / csrc/attention_bwd.cu, with a PyTorch reference used on CPU and as the
test oracle.

Tensors are passed as ``[b, s, heads, hd]`` views with arbitrary batch / sequence / head strides
(the head dim contiguous), so the q / k / v slices of the fused QKV projection output are consumed
in place.  Counterpart of megatron/model/transformer.py:573-690.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from .gemm import LAUNCHES


def alibi_slopes(n_heads: int) -> torch.Tensor:
    """Per-head ALiBi slopes (megatron/model/positional_embeddings.py:146-167)."""
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(n_heads).is_integer():
        s = pow2(n_heads)
    else:
        c = 2 ** math.floor(math.log2(n_heads))
        s = pow2(c) + pow2(2 * c)[0::2][: n_heads - c]
    return torch.tensor(s, dtype=torch.float32)


_M32 = 0xFFFFFFFF


def _mul32(x, c):
    """(x * c) mod 2^32 on int64 tensors holding 32-bit values, without overflowing 64 bits."""
    return (x * (c & 0xFFFF) + (((x * (c >> 16)) & 0xFFFF) << 16)) & _M32


def _mix32(x):
    x = x ^ (x >> 16)
    x = _mul32(x, 0x7FEB352D)
    x = x ^ (x >> 15)
    x = _mul32(x, 0x846CA68B)
    return x ^ (x >> 16)


def dropout_threshold(p: float) -> int:
    """The kernels quantise the dropout probability to 1/256: keep iff hash byte >= this threshold."""
    return min(255, int(p * 256.0 + 0.5))


def dropout_keep_mask(b: int, h: int, sq: int, sk: int, p: float, seed: int, device="cpu") -> torch.Tensor:
    """The attention kernels' dropout mask as a bool tensor [b, h, sq, sk] (True = kept): the PyTorch
    statement of ``dropout_patch`` / ``dropout_keep`` in csrc/ptx.cuh.  A pure function of
    (seed, batch * h + head, q, k), so forward and backward of any implementation agree on it."""
    thr = dropout_threshold(p)
    seed &= 0xFFFFFFFFFFFFFFFF
    seed_lo, seed_hi = seed & _M32, seed >> 32
    q = torch.arange(sq, device=device, dtype=torch.int64)[:, None]
    k = torch.arange(sk, device=device, dtype=torch.int64)[None, :]
    x = _mix32((((q >> 1) << 16) | (k >> 1)) ^ seed_lo)                       # [sq, sk]
    bh = torch.arange(b * h, device=device, dtype=torch.int64)[:, None, None]
    patch = _mix32((x[None] + _mul32(bh, 0x9E3779B9) + seed_hi) & _M32)       # [b*h, sq, sk]
    byte = (patch >> ((((q & 1) << 1) | (k & 1)) * 8)[None]) & 0xFF
    return (byte >= thr).view(b, h, sq, sk)


_DROPOUT_CALLS = {"n": 0}


def next_dropout_seed(stream_id: int = 0) -> int:
    """A fresh 64-bit seed per dropout call: the process seed, a call counter (saved and replayed by activation
    checkpointing, parallel/random.py) and ``stream_id`` (the tensor-parallel rank: ranks hold different heads)."""
    _DROPOUT_CALLS["n"] += 1
    return (torch.initial_seed() * 0x9E3779B97F4A7C15 + _DROPOUT_CALLS["n"] * 0xD1B54A32D192ED03
            + stream_id * 0x8CB92BA72F3D8DD7) & 0xFFFFFFFFFFFFFFFF


class BlockLayout:
    """A block-sparse attention pattern: ``allowed`` bool [nb, nb] (query block attends to key block, before
    causality; one layout for all heads) over square blocks of ``block`` tokens (16, 32, 64 or 128 for the CUDA
    kernels, which skip key tiles without a live block and mask the rest per sub-block).  Builds and caches the two
    byte tables the kernels read for a given (sq, sk) on a device."""

    def __init__(self, allowed: torch.Tensor, block: int):
        assert allowed.dim() == 2 and allowed.shape[0] == allowed.shape[1] and allowed.dtype == torch.bool
        self.allowed, self.block = allowed.cpu(), int(block)
        self._tables = {}

    @property
    def kernel_ok(self):
        return self.block in (16, 32, 64, 128)

    def token_allowed(self, sq: int, sk: int, device="cpu") -> torch.Tensor:
        """bool [sq, sk]: query i (at position i + sk - sq) may attend to key j."""
        nb = self.allowed.shape[0]
        qb = ((torch.arange(sq) + (sk - sq)) // self.block).clamp(max=nb - 1)
        kb = (torch.arange(sk) // self.block).clamp(max=nb - 1)
        return self.allowed[qb][:, kb].to(device)

    def tables(self, sq: int, sk: int, device):
        """(rows uint8 [sq, ceil(sk / 128)], any uint8 [ceil(sq / 128), ceil(sk / 128)]) for the kernels."""
        key = (sq, sk, str(device))
        if key not in self._tables:
            sub = 128 // self.block                         # key sub-blocks per 128-key tile
            nkt = (sk + 127) // 128
            nb = self.allowed.shape[0]
            qb = ((torch.arange(sq) + (sk - sq)) // self.block).clamp(max=nb - 1)
            kb = torch.arange(nkt * sub)
            live = self.allowed[qb][:, kb.clamp(max=nb - 1)] & (kb < (sk + self.block - 1) // self.block)[None, :]
            live = live.view(sq, nkt, sub).to(torch.int32)
            rows = (live << torch.arange(sub, dtype=torch.int32)[None, None, :]).sum(-1).to(torch.uint8)
            pad = (-sq) % 128
            anyt = torch.nn.functional.pad(rows, (0, 0, 0, pad)).view(-1, 128, nkt).amax(dim=1)
            self._tables[key] = (rows.contiguous().to(device), (anyt != 0).to(torch.uint8).contiguous().to(device))
        return self._tables[key]


def attention_reference(q, k, v, *, scale=None, causal=True, window: int = -1, alibi=None, dropout_p: float = 0.0,
                        seed: int = 0, block_layout: BlockLayout | None = None):
    """Plain PyTorch attention in fp32. q [b,sq,h,d], k/v [b,sk,hk,d] -> ([b,sq,h,d], lse [b,h,sq]).
    ``dropout_p`` > 0 applies the kernels' own mask (``dropout_keep_mask``) to the normalised probabilities."""
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qf, kf, vf = q.float(), k.float(), v.float()
    if hk != h:
        kf = kf.repeat_interleave(h // hk, dim=2)
        vf = vf.repeat_interleave(h // hk, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    qpos = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
    kpos = torch.arange(sk, device=q.device)[None, :]
    if alibi is not None:
        s = s + alibi.to(s.device).float()[None, :, None, None] * (kpos - qpos).float()[None, None]
    dead = torch.zeros(sq, sk, dtype=torch.bool, device=q.device)
    if causal:
        dead |= kpos > qpos
    if window is not None and window >= 0:
        dead |= kpos < qpos - window
    if block_layout is not None:
        dead |= ~block_layout.token_allowed(sq, sk, q.device)
    s = s.masked_fill(dead[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    if dropout_p > 0:
        keep = dropout_keep_mask(b, h, sq, sk, dropout_p, seed, q.device)
        p = p * keep * (256.0 / (256 - dropout_threshold(dropout_p)))
    o = torch.einsum("bhqk,bkhd->bqhd", p, vf)
    return o.to(q.dtype), lse


def _strides_bhs(t):
    # tensor is [b, s, h, d] -> (batch, head, seq) element strides
    return t.stride(0), t.stride(2), t.stride(1)


def _layout_args(layout, sq, sk, device):
    """(rows pointer, any pointer, block size) of a block layout for the kernels; (None, None, 0) without one.
    The tensors are returned too so that they stay alive across the launch."""
    if layout is None:
        return None, None, 0, None
    rows, anyt = layout.tables(sq, sk, device)
    return _lib.ptr(rows), _lib.ptr(anyt), layout.block, (rows, anyt)


def _fwd(q, k, v, scale, causal, window, alibi, dropout_p=0.0, seed=0, layout=None):
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    o = torch.empty((b, sq, h, d), device=q.device, dtype=q.dtype)
    # base-2 log-sum-exp, rows padded to a multiple of 128 with +inf (the backward reads whole
    # 128-row blocks of it; +inf makes the padding contribute zero probability)
    sq_pad = (sq + 127) // 128 * 128
    lse = torch.full((b, h, sq_pad), float("inf"), device=q.device, dtype=torch.float32)
    LAUNCHES["n"] += 1
    rows, anyt, blk, _keep = _layout_args(layout, sq, sk, q.device)
    _lib.check(_lib.lib(q).nx_flash_attn_fwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(alibi),
        b, h, hk, sq, sk, d, *_strides_bhs(q), *_strides_bhs(k), *_strides_bhs(v), *_strides_bhs(o),
        float(scale), int(causal), int(window), float(dropout_p), int(seed), rows, anyt, blk, _lib.stream()),
        "nx_flash_attn_fwd")
    return o, lse


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, window, alibi, dropout_p=0.0, seed=0, layout=None):
        o, lse = _fwd(q, k, v, scale, causal, window, alibi, dropout_p, seed, layout)
        ctx.save_for_backward(q, k, v, o, lse, alibi)
        ctx.scale, ctx.causal, ctx.window, ctx.dropout, ctx.layout = scale, causal, window, (dropout_p, seed), layout
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, alibi = ctx.saved_tensors
        b, sq, h, d = q.shape
        sk, hk = k.shape[1], k.shape[2]
        if do.stride(3) != 1 or any(s % 8 for s in do.stride()[:3]):
            do = do.contiguous()
        dq = torch.empty((b, sq, h, d), device=q.device, dtype=q.dtype)
        dk = torch.empty((b, sk, hk, d), device=q.device, dtype=q.dtype)
        dv = torch.empty((b, sk, hk, d), device=q.device, dtype=q.dtype)
        # (rows beyond the sequence exist only when it is not a multiple of the 128-row tile: only then a fill)
        delta = (torch.empty if lse.shape[-1] == sq else torch.zeros)(lse.shape, device=q.device, dtype=torch.float32)
        LAUNCHES["n"] += 3
        rows, anyt, blk, _keep = _layout_args(ctx.layout, sq, sk, q.device)
        _lib.check(_lib.lib(q).nx_flash_attn_bwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse),
            _lib.ptr(delta), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(alibi),
            b, h, hk, sq, sk, d, *_strides_bhs(q), *_strides_bhs(k), *_strides_bhs(v), *_strides_bhs(o),
            *_strides_bhs(do), *_strides_bhs(dq), *_strides_bhs(dk), *_strides_bhs(dv),
            float(ctx.scale), int(ctx.causal), int(ctx.window), float(ctx.dropout[0]), int(ctx.dropout[1]),
            rows, anyt, blk, _lib.stream()), "nx_flash_attn_bwd")
        return dq, dk, dv, None, None, None, None, None, None, None


def flash_attention(q, k, v, *, scale: float | None = None, causal: bool = True, window: int = -1,
                    alibi: torch.Tensor | None = None, dropout_p: float = 0.0, seed: int | None = None,
                    block_layout: BlockLayout | None = None) -> torch.Tensor:
    """q [b,sq,h,d]; k, v [b,sk,hk,d] (h % hk == 0). Query i sits at position i + (sk - sq) (cached decoding:
    sq new tokens against sk keys).  ``dropout_p`` > 0: dropout on the probabilities, mask regenerated in the
    backward from ``seed`` (default: a fresh one per call).  ``block_layout``: block-sparse pattern (key tiles
    without a live block are skipped)."""
    if dropout_p > 0 and seed is None:
        seed = next_dropout_seed()
    seed = seed or 0
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    window = -1 if window is None else int(window)
    if q.is_cuda:
        if q.dtype not in _lib.H16 or d % 8 or d > 128:
            raise _lib.KernelError(f"flash_attention: CUDA path needs bf16 and head dim % 8 == 0, <= 128 (got {q.dtype}, {d})")
        fix = lambda t: t if (t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0) else t.contiguous()
        if alibi is not None:
            alibi = alibi.to(device=q.device, dtype=torch.float32).contiguous()
        if block_layout is not None and not block_layout.kernel_ok:
            raise _lib.KernelError(f"flash_attention: block-sparse layouts need blocks of 16, 32, 64 or 128 tokens "
                                   f"(got {block_layout.block})")
        return _FlashAttnFn.apply(fix(q), fix(k), fix(v), scale, causal, window, alibi, float(dropout_p), seed,
                                  block_layout)
    return attention_reference(q, k, v, scale=scale, causal=causal, window=window, alibi=alibi, dropout_p=dropout_p,
                               seed=seed, block_layout=block_layout)[0]


def flash_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, *, scale: float | None = None, causal: bool = True,
                           window: int = -1, alibi: torch.Tensor | None = None, dropout_p: float = 0.0,
                           seed: int | None = None) -> torch.Tensor:
    """Attention over sequences packed back to back (the ``flash_attn_varlen_func`` calling convention the reference
    uses for cached inference, megatron/model/transformer.py:636-664): ``q`` [total_q, h, d], ``k`` / ``v``
    [total_k, hk, d]; ``cu_seqlens_*``: cumulative lengths (``[0, l0, l0 + l1, ...]``, a list or an int tensor).
    Sequence i attends only to itself; its queries sit at the END of its keys when the lengths differ (decoding).
    Each sequence is one launch of the flash kernel on a strided view of the packed tensors, so memory stays linear
    in the sequence length and there is no padding."""
    cq = cu_seqlens_q.tolist() if torch.is_tensor(cu_seqlens_q) else list(cu_seqlens_q)
    ck = cu_seqlens_k.tolist() if torch.is_tensor(cu_seqlens_k) else list(cu_seqlens_k)
    assert len(cq) == len(ck) and cq[0] == 0 and ck[0] == 0 and cq[-1] == q.shape[0] and ck[-1] == k.shape[0]
    if dropout_p > 0 and seed is None:
        seed = next_dropout_seed()
    outs = []
    for i in range(len(cq) - 1):
        qi, ki, vi = q[cq[i]:cq[i + 1]], k[ck[i]:ck[i + 1]], v[ck[i]:ck[i + 1]]
        if qi.shape[0] == 0:
            continue
        outs.append(flash_attention(qi.unsqueeze(0), ki.unsqueeze(0), vi.unsqueeze(0), scale=scale, causal=causal,
                                    window=window, alibi=alibi, dropout_p=dropout_p,
                                    seed=None if seed is None else (seed + i) & 0xFFFFFFFFFFFFFFFF).squeeze(0))
    return torch.cat(outs, dim=0) if outs else q.new_zeros(q.shape)
