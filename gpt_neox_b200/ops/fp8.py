"""FP8 linear layers with per-tensor delayed scaling (csrc/gemm_fp8_tcgen05.cu).

Forward and both backward GEMMs run on ``tcgen05.mma.kind::f8f6f4``: activations and weights in e4m3,
gradients in e5m2 (the "hybrid" format), fp32 accumulation, bf16 outputs, weight gradients accumulated in
fp32 into ``weight.main_grad`` when the engine provides it.  Scales follow the delayed-scaling recipe the
reference configures through Transformer Engine (megatron/model/transformer_engine.py:633-670): each
tensor role keeps a history of absolute maxima; the scale used at step t is ``fp8_max / (2^margin *
max(history))`` computed from steps before t, and the amax observed at step t is recorded for later.
All of this state lives on the device: no host synchronisation per step.

Both operands of the fp8 MMA are K-major here, so the backward GEMMs consume transposed fp8 copies that
the quantisation kernel writes in the same pass as the straight copy.
"""
from __future__ import annotations

import torch

from . import _lib
from .gemm import LAUNCHES

E4M3_MAX, E5M2_MAX = 448.0, 57344.0


class Fp8TensorMeta:
    """Scale state of one tensor role (input, weight or output-gradient of one layer)."""

    def __init__(self, device, e5m2=False, history=16, margin=0, algo="max"):
        self.fp8_max = E5M2_MAX if e5m2 else E4M3_MAX
        self.e5m2, self.margin, self.algo = e5m2, margin, algo
        self.scale = torch.ones(1, device=device, dtype=torch.float32)
        self.amax = torch.zeros(1, device=device, dtype=torch.float32)            # written by the kernel
        self.history = torch.zeros(history, device=device, dtype=torch.float32)

    def roll(self):
        """Record the amax observed since the last call and derive the next scale (device-side ops)."""
        self.history = torch.roll(self.history, 1)
        self.history[0] = self.amax[0]
        self.amax.zero_()
        m = self.history[0] if self.algo == "most_recent" else self.history.max()
        new = self.fp8_max / (m * (2.0 ** self.margin))
        self.scale = torch.where((m > 0) & torch.isfinite(new), new, self.scale).reshape(1)


class Fp8LinearMeta:
    def __init__(self, device, history=16, margin=0, algo="max", hybrid=True, fp8_wgrad=True):
        self.x = Fp8TensorMeta(device, False, history, margin, algo)
        self.w = Fp8TensorMeta(device, False, history, margin, algo)
        self.g = Fp8TensorMeta(device, hybrid, history, margin, algo)      # hybrid: e5m2 gradients
        self.fp8_wgrad = fp8_wgrad

    @classmethod
    def from_args(cls, neox_args, device):
        return cls(device, history=max(1, neox_args.te_fp8_amax_history_len), margin=neox_args.te_fp8_margin,
                   algo=neox_args.te_fp8_amax_compute_algo, hybrid=neox_args.te_fp8_format == "hybrid",
                   fp8_wgrad=bool(neox_args.te_fp8_wgrad))

    def roll(self):
        self.x.roll(), self.w.roll(), self.g.roll()
        self._w_cache = None              # new scale, new weights: the quantised weight copies are stale


def quantize(x2, meta: Fp8TensorMeta, transpose=False):
    """bf16 [rows, cols] -> (fp8 [rows, cols], fp8 [cols, rows] or None) as uint8 tensors; updates meta.amax."""
    rows, cols = x2.shape
    out = torch.empty((rows, cols), device=x2.device, dtype=torch.uint8)
    out_t = torch.empty((cols, rows), device=x2.device, dtype=torch.uint8) if transpose else None
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib().nx_fp8_quantize(_lib.ptr(x2), x2.stride(0), _lib.ptr(meta.scale), _lib.ptr(out), cols,
                                          _lib.ptr(out_t), rows, _lib.ptr(meta.amax), rows, cols, int(meta.e5m2),
                                          _lib.stream()), "nx_fp8_quantize")
    return out, out_t


def gemm_fp8(a8, b8, alpha, *, a_e5m2=False, b_e5m2=False, bias=None, out=None, accumulate=False):
    """C[M,N] = alpha * a8[M,K] @ b8[N,K]^T (+ bias); bf16 result, or fp32 into ``out`` (optionally +=)."""
    M, K = a8.shape
    N = b8.shape[0]
    out_f32 = out is not None and out.dtype == torch.float32
    if out is None:
        out = torch.empty((M, N), device=a8.device, dtype=torch.bfloat16)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib().nx_gemm_fp8(_lib.ptr(a8), _lib.ptr(b8), _lib.ptr(out), M, N, K, a8.stride(0), b8.stride(0),
                                      out.stride(0), int(a_e5m2), int(b_e5m2), _lib.ptr(alpha), _lib.ptr(bias),
                                      int(out_f32), int(accumulate), _lib.stream()), "nx_gemm_fp8")
    return out


def _delayed_weight(weight, meta: "Fp8LinearMeta", transpose: bool):
    """The quantised weight (and its transpose) of this optimizer step.  Under delayed scaling the weight's scale
    changes only when the history rolls (once per step) and the weight itself only in the optimizer step, so every
    micro-batch of a step reuses the first one's copies.  ``Fp8LinearMeta.roll`` drops them."""
    key = (weight.data_ptr(), weight._version, bool(transpose))
    hit = getattr(meta, "_w_cache", None)
    if hit is None or hit[0] != key:
        hit = (key, quantize(weight, meta.w, transpose=transpose))
        meta._w_cache = hit
    return hit[1]


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, meta: Fp8LinearMeta):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        need_wgrad = weight.requires_grad
        x8, x8t = quantize(x2, meta.x, transpose=need_wgrad and meta.fp8_wgrad)
        w8, w8t = _delayed_weight(weight, meta, transpose=x.requires_grad)
        alpha = 1.0 / (meta.x.scale * meta.w.scale)
        y = gemm_fp8(x8, w8, alpha, bias=bias)
        ctx.save_for_backward(x8t, w8t, meta.x.scale.clone(), meta.w.scale.clone(),
                              x2 if (need_wgrad and not meta.fp8_wgrad) else None)
        ctx.meta, ctx.weight, ctx.has_bias, ctx.x_shape = meta, weight, bias is not None, x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x8t, w8t, sx, sw, x_bf16 = ctx.saved_tensors
        meta, weight = ctx.meta, ctx.weight
        g2 = gy.reshape(-1, gy.shape[-1])
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        g8, g8t = quantize(g2, meta.g, transpose=x8t is not None)
        gx = gw = gb = None
        if w8t is not None:
            gx = gemm_fp8(g8, w8t, 1.0 / (meta.g.scale * sw), a_e5m2=meta.g.e5m2).view(ctx.x_shape)     # dY [M,N] x W^T[K,N]^T
        if x8t is not None:
            mg = getattr(weight, "main_grad", None)
            alpha = 1.0 / (meta.g.scale * sx)
            if mg is not None and mg.dtype == torch.float32:
                gemm_fp8(g8t, x8t, alpha, a_e5m2=meta.g.e5m2, out=mg, accumulate=True)                  # dY^T [N,M] x X^T[K,M]^T
            else:
                gw = gemm_fp8(g8t, x8t, alpha, a_e5m2=meta.g.e5m2)
                if mg is not None:
                    mg.add_(gw.to(mg.dtype))
                    gw = None
        if x_bf16 is not None:
            from .gemm import wgrad
            gw = wgrad(g2, x_bf16, weight)                       # te_fp8_wgrad = false: bf16 weight gradient
        if ctx.has_bias:
            from .elementwise import colsum
            gb = colsum(g2)
        return gx, gw, gb, None


def fp8_linear(x, weight, bias, meta: Fp8LinearMeta):
    """``F.linear`` with fp8 tensor-core GEMMs. Shapes: tokens % 8 == 0, in/out features % 16 == 0."""
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        raise _lib.KernelError("fp8_linear needs CUDA bf16 activations")
    return _Fp8LinearFn.apply(x, weight, bias, meta)


def dequantize_reference(q8, scale, e5m2=False):
    """uint8 fp8 bit patterns -> fp32 values / scale (test helper)."""
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    return q8.view(dt).float() / scale


# ---------------------------------------------------------------------------------------------------------------
# Block-scaled fp8 (MXFP8): one power-of-two scale per 32 consecutive elements of a row, applied by the tensor core
# (csrc/gemm_mxfp8_tcgen05.cu).  No amax history and no per-tensor scale: every tensor is quantised from its own
# values when it is used.  Scale layout: uint32 words [ceil(cols / 128)][rows padded to 128], word = the ue8m0 bytes of
# four consecutive 32-element groups of one row.
# ---------------------------------------------------------------------------------------------------------------
def _pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def mxfp8_quantize(x2: torch.Tensor, e5m2: bool = False):
    """16-bit [rows, cols] (cols % 32 == 0) -> (fp8 bytes [rows, cols] uint8, scale words [ceil(cols/128), pad128(rows)]
    int32)."""
    rows, cols = x2.shape
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    out = torch.empty((rows, cols), device=x2.device, dtype=torch.uint8)
    sf = torch.full(((cols + 127) // 128, _pad128(rows)), 0x7F7F7F7F, device=x2.device, dtype=torch.int32)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(x2).nx_mxfp8_quantize(_lib.ptr(x2), x2.stride(0), _lib.ptr(out), cols, _lib.ptr(sf), sf.stride(0),
                                              rows, cols, int(e5m2), _lib.stream()), "nx_mxfp8_quantize")
    return out, sf


def mxfp8_quantize_reference(x2: torch.Tensor, e5m2: bool = False):
    """The quantiser in plain PyTorch (any device): same bytes and scale words as the kernel."""
    rows, cols = x2.shape
    fmax = E5M2_MAX if e5m2 else E4M3_MAX
    g = x2.float().reshape(rows, cols // 32, 32)
    amax = g.abs().amax(-1)
    mant, ex = torch.frexp(amax / fmax)                                   # amax / fmax = mant * 2^ex, mant in [0.5, 1)
    e = torch.where(mant == 0.5, ex - 1, ex).clamp(-127, 127)             # ceil(log2(.))
    e = torch.where(amax > 0, e, torch.zeros_like(e))
    q = (g * torch.exp2(-e.float()).unsqueeze(-1)).clamp(-fmax, fmax)
    q8 = q.to(torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn).view(torch.uint8).reshape(rows, cols)
    nkb = (cols + 127) // 128
    by = torch.full((nkb, _pad128(rows), 4), 127, dtype=torch.int32, device=x2.device)
    eb = (e + 127).to(torch.int32)                                        # [rows, groups]
    ngr = cols // 32
    padded = torch.full((rows, nkb * 4), 127, dtype=torch.int32, device=x2.device)
    padded[:, :ngr] = eb
    by[:, :rows, :] = padded.reshape(rows, nkb, 4).permute(1, 0, 2)
    words = by[..., 0] | (by[..., 1] << 8) | (by[..., 2] << 16) | (by[..., 3] << 24)
    return q8, words.to(torch.int32)


def mxfp8_dequantize_reference(q8: torch.Tensor, sf: torch.Tensor, e5m2: bool = False) -> torch.Tensor:
    """fp8 bytes + scale words -> fp32 values (test helper)."""
    rows, cols = q8.shape
    vals = q8.view(torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn).float()
    nkb = sf.shape[0]
    w = sf[:, :rows].to(torch.int64) & 0xFFFFFFFF                         # [nkb, rows]
    by = torch.stack([(w >> (8 * i)) & 0xFF for i in range(4)], dim=-1)   # [nkb, rows, 4]
    e = (by.permute(1, 0, 2).reshape(rows, nkb * 4)[:, :cols // 32] - 127).float()
    return (vals.reshape(rows, cols // 32, 32) * torch.exp2(e).unsqueeze(-1)).reshape(rows, cols)


def gemm_mxfp8(a8, sfa, b8, sfb, *, a_e5m2=False, b_e5m2=False, bias=None, out=None, accumulate=False, alpha=None,
               out_dtype=torch.bfloat16, tile: int = 0):
    """C[M,N] = (a8 with its block scales)[M,K] @ (b8 with its block scales)[N,K]^T (+ bias); 16-bit result, or fp32 into
    ``out`` (optionally +=).  ``tile``: tile width of the kernel (0 = its own choice; 128 / 192 / 224 / 256)."""
    M, K = a8.shape
    N = b8.shape[0]
    out_f32 = out is not None and out.dtype == torch.float32
    if out is None:
        out = torch.empty((M, N), device=a8.device, dtype=out_dtype)
    like = out if not out_f32 else (bias if bias is not None else torch.empty(0, dtype=out_dtype))
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(like).nx_gemm_mxfp8(_lib.ptr(a8), _lib.ptr(b8), _lib.ptr(out), M, N, K, a8.stride(0), b8.stride(0),
                                            out.stride(0), _lib.ptr(sfa), _lib.ptr(sfb), sfa.stride(0), sfb.stride(0),
                                            int(a_e5m2), int(b_e5m2), _lib.ptr(alpha), _lib.ptr(bias), int(out_f32),
                                            int(accumulate), int(tile), _lib.stream()), "nx_gemm_mxfp8")
    return out


def mxfp8_quantize_dual(x2: torch.Tensor, e5m2: bool = False):
    """One read of x [rows, cols] (both multiples of 32), both quantised forms: (q [rows, cols], sf) with the scale
    blocks along the columns, and (q_t [cols, rows], sf_t) = the same for x transposed (blocks along the rows of x)."""
    rows, cols = x2.shape
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    dev = x2.device
    out = torch.empty((rows, cols), device=dev, dtype=torch.uint8)
    out_t = torch.empty((cols, rows), device=dev, dtype=torch.uint8)
    sf = torch.full(((cols + 127) // 128, _pad128(rows)), 0x7F7F7F7F, device=dev, dtype=torch.int32)
    sf_t = torch.full(((rows + 127) // 128, _pad128(cols)), 0x7F7F7F7F, device=dev, dtype=torch.int32)
    LAUNCHES["n"] += 1
    _lib.check(_lib.lib(x2).nx_mxfp8_quantize_dual(_lib.ptr(x2), x2.stride(0), _lib.ptr(out), cols, _lib.ptr(sf),
                                                   sf.stride(0), _lib.ptr(out_t), rows, _lib.ptr(sf_t), sf_t.stride(0),
                                                   rows, cols, int(e5m2), _lib.stream()), "nx_mxfp8_quantize_dual")
    return out, sf, out_t, sf_t


#: quantised weights are reused by every micro-batch of an optimizer step: id(weight) -> (step generation, data pointer,
#: tensor version, the four tensors of mxfp8_quantize_dual).  The engine bumps the generation after every optimizer step
#: (its fused update writes the weights through raw pointers, which no tensor version records).
_MX_WEIGHTS: dict = {}
_MX_GENERATION = {"n": 0}


def mxfp8_new_step():
    _MX_GENERATION["n"] += 1
    if len(_MX_WEIGHTS) > 4096:
        _MX_WEIGHTS.clear()


def _mx_weight(weight):
    key = (_MX_GENERATION["n"], weight.data_ptr(), weight._version)
    hit = _MX_WEIGHTS.get(id(weight))
    if hit is None or hit[0] != key:
        hit = (key, mxfp8_quantize_dual(weight.detach()))
        _MX_WEIGHTS[id(weight)] = hit
    return hit[1]


class _MxFp8LinearFn(torch.autograd.Function):
    """y = x W^T (+ b) with all three GEMMs block-scaled.  Every GEMM contracts over the dimension its operands were
    quantised along: forward x [M,K] and W [N,K] along K; input gradient dY [M,N] and W^T [K,N] along N; weight
    gradient dY^T [N,M] and x^T [K,M] along M.  The transposed forms come out of the same quantiser pass as the
    straight ones (one read of x, of dY and -- once per optimizer step -- of W)."""

    @staticmethod
    def forward(ctx, x, weight, bias, hybrid):
        x2 = x.reshape(-1, x.shape[-1])
        need_wgrad = ctx.needs_input_grad[1]
        w8, sw, wt8, swt = _mx_weight(weight)
        if need_wgrad and x2.shape[0] % 32 == 0:
            x8, sx, xt8, sxt = mxfp8_quantize_dual(x2)
        else:
            (x8, sx), xt8, sxt = mxfp8_quantize(x2), None, None
        y = gemm_mxfp8(x8, sx, w8, sw, bias=bias, out_dtype=x.dtype)
        ctx.save_for_backward(xt8, sxt, wt8, swt, x2 if (need_wgrad and xt8 is None) else None)
        ctx.weight, ctx.bias, ctx.has_bias, ctx.x_shape, ctx.hybrid = weight, bias, bias is not None, x.shape, hybrid
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        xt8, sxt, wt8, swt, x2 = ctx.saved_tensors
        weight = ctx.weight
        g2 = gy.reshape(-1, gy.shape[-1])
        e5 = bool(ctx.hybrid)
        gx = gw = gb = None
        need_gw = ctx.needs_input_grad[1]
        if need_gw and g2.shape[0] % 32 == 0:
            g8, sg, gt8, sgt = mxfp8_quantize_dual(g2, e5m2=e5)
        else:
            g8, sg = mxfp8_quantize(g2, e5m2=e5)
            gt8, sgt = mxfp8_quantize(g2.t().contiguous(), e5m2=e5) if need_gw else (None, None)
        if ctx.needs_input_grad[0]:
            gx = gemm_mxfp8(g8, sg, wt8, swt, a_e5m2=e5, out_dtype=gy.dtype).view(ctx.x_shape)
        if need_gw:
            if xt8 is None:
                xt8, sxt = mxfp8_quantize(x2.t().contiguous())
            mg = getattr(weight, "main_grad", None)
            if mg is not None and mg.dtype == torch.float32:
                gemm_mxfp8(gt8, sgt, xt8, sxt, a_e5m2=e5, out=mg, accumulate=True, out_dtype=gy.dtype)
            else:
                gw = gemm_mxfp8(gt8, sgt, xt8, sxt, a_e5m2=e5, out_dtype=gy.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .elementwise import bias_grad
            gb = bias_grad(g2.contiguous(), ctx.bias)
        return gx, gw, gb, None


def mxfp8_linear(x, weight, bias=None, hybrid: bool = True):
    """``F.linear`` on block-scaled fp8 tensor-core GEMMs (tokens, in and out features multiples of 32)."""
    if not (x.is_cuda and x.dtype in _lib.H16):
        raise _lib.KernelError("mxfp8_linear needs CUDA bf16 / fp16 activations")
    return _MxFp8LinearFn.apply(x, weight, bias, hybrid)
