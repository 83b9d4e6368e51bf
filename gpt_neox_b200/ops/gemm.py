"""Dense bf16 GEMM on tcgen05 tensor cores, with fused epilogues, and the autograd
``linear`` built on it.

Counterpart of the cuBLAS ``F.linear`` calls of the reference
(megatron/mpu/layers.py:576,773; megatron/model/transformer.py:1240-1242) and of its
torch.jit bias+GeLU fusion (megatron/model/activations.py:78-112).

On CPU tensors (tests, the gloo plumbing runs) the same functions compute with plain
PyTorch in the tensor's dtype; that path is the numerical oracle of the CUDA kernels.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

EPI_BIAS = 1
EPI_GELU_ERF = 2
EPI_GELU_TANH = 4
EPI_AUX_OUT = 8
EPI_DGELU_ERF = 16
EPI_DGELU_TANH = 32
EPI_RESIDUAL = 64
EPI_ACCUM = 128
EPI_OUT_F32 = 256
EPI_SCALE = 512
EPI_AUX_DERIV = 1024       # aux_out receives gelu'(pre-activation) instead of the pre-activation
EPI_MUL_AUX = 2048         # multiply by dgelu_aux as it is (a stored derivative)

#: counts launches of this library's kernels (read by bench.py for its ``gpu_launches`` claim)
LAUNCHES = {"n": 0}
#: use the CTA-pair GEMM kernel (csrc/gemm2_tcgen05.cu) for problems of at least one 256 x 256 tile
PAIR_GEMM = {"on": __import__("os").environ.get("NEOX_GEMM_2CTA", "1") == "1"}


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0 or (x2.data_ptr() % 16) != 0:
        x2 = x2.contiguous()
    return x2


def aux_flags(gelu, aux_out, aux_deriv, dgelu_aux, dgelu) -> int:
    """Epilogue flags of the auxiliary operands.  ``aux_deriv``: ``aux_out`` receives gelu'(pre-activation)
    instead of the pre-activation; the matching backward GEMM passes it as ``dgelu_aux`` with ``dgelu="mul"``,
    so its epilogue is one multiply instead of an erf / exp evaluation per element."""
    flags = 0
    if aux_out is not None:
        flags |= EPI_AUX_OUT
        if aux_deriv:
            assert gelu is not None, "aux_deriv needs a GeLU epilogue"
            flags |= EPI_AUX_DERIV
    if dgelu_aux is not None:
        flags |= {"tanh": EPI_DGELU_TANH, "mul": EPI_MUL_AUX}.get(dgelu, EPI_DGELU_ERF)
    return flags


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         bias: torch.Tensor | None = None, gelu: str | None = None,
         aux_out: torch.Tensor | None = None, dgelu_aux: torch.Tensor | None = None,
         dgelu: str | None = None, residual: torch.Tensor | None = None,
         out: torch.Tensor | None = None, accumulate: bool = False,
         out_dtype: torch.dtype | None = None, alpha: float | None = None,
         aux_deriv: bool = False) -> torch.Tensor:
    """``C = epilogue(op(a) @ op(b))`` with 2-D row-major 16-bit operands (bf16 or fp16, both the same dtype).

    ``trans_a=False``: a is [M,K]; ``True``: a is [K,M].
    ``trans_b=False``: b is [N,K] (weight layout); ``True``: b is [K,N].
    Epilogue order: scale, +bias, store ``aux_out`` (the pre-activation, or its GeLU derivative with
    ``aux_deriv``), ×gelu'(``dgelu_aux``) (``dgelu="mul"``: × ``dgelu_aux`` itself), GeLU, +residual,
    (+= out if ``accumulate``).
    """
    assert a.is_cuda and a.dtype in _lib.H16 and b.dtype == a.dtype, (a.dtype, b.dtype)
    if trans_a:
        K, M = a.shape
    else:
        M, K = a.shape
    if trans_b:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    assert a.stride(1) == 1 and b.stride(1) == 1
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or a.dtype)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1
    flags = 0
    if out.dtype == torch.float32:
        flags |= EPI_OUT_F32
    else:
        assert out.dtype == a.dtype, (out.dtype, a.dtype)
    if bias is not None:
        assert bias.dtype == a.dtype and bias.numel() == N
        flags |= EPI_BIAS
    if gelu is not None:
        flags |= EPI_GELU_TANH if gelu == "tanh" else EPI_GELU_ERF
    ld_aux = 0
    for t in (aux_out, dgelu_aux, residual):
        if t is not None:
            assert t.shape == (M, N) and t.stride(1) == 1 and t.dtype == a.dtype
            assert ld_aux in (0, t.stride(0)), "aux tensors must share one leading dimension"
            ld_aux = t.stride(0)
    flags |= aux_flags(gelu, aux_out, aux_deriv, dgelu_aux, dgelu)
    if residual is not None:
        flags |= EPI_RESIDUAL
    if accumulate:
        flags |= EPI_ACCUM
    if alpha is not None:
        flags |= EPI_SCALE
    L = _lib.lib(a)
    LAUNCHES["n"] += 1
    fn, name = L.nx_gemm_bf16, "nx_gemm_bf16"
    if PAIR_GEMM["on"] and M >= 256 and N >= 256:
        fn, name = L.nx_gemm2_bf16, "nx_gemm2_bf16"      # CTA-pair kernel (cta_group::2, 256 x 256 tiles)
    _lib.check(fn(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(trans_a), int(trans_b), _lib.ptr(bias), _lib.ptr(dgelu_aux), _lib.ptr(aux_out),
        _lib.ptr(residual), ld_aux, flags, float(alpha if alpha is not None else 1.0),
        _lib.stream()), name)
    return out


class _LinearFn(torch.autograd.Function):
    """y = x @ W^T (+ b) with the three GEMMs (forward, dgrad, wgrad) on tcgen05.

    ``W.main_grad`` (fp32, optional): when present the weight gradient is accumulated into it
    by the wgrad epilogue and ``None`` is returned for W — the fused gradient-accumulation
    path used by the ZeRO engine.
    """

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = _as_2d(x)
        y = gemm(x2, weight, bias=bias)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias, ctx.bias = bias is not None, bias
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, weight = ctx.saved_tensors
        gy2 = _as_2d(gy)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = gemm(gy2, weight, trans_b=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw = wgrad(gy2, x2, weight)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .elementwise import bias_grad
            gb = bias_grad(gy2, ctx.bias)
        return gx, gw, gb


def wgrad(gy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor):
    """dW[N,K] = gy2[M,N]^T @ x2[M,K]; accumulates into ``weight.main_grad`` when it exists."""
    mg = getattr(weight, "main_grad", None)
    if mg is not None:
        gemm(gy2, x2, trans_a=True, trans_b=True, out=mg, accumulate=True)
        return None
    return gemm(gy2, x2, trans_a=True, trans_b=True)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear`` on the tcgen05 GEMM for CUDA bf16 / fp16 tensors; PyTorch on CPU (oracle path)."""
    if x.is_cuda and x.dtype in _lib.H16:
        return _LinearFn.apply(x, weight, bias)
    if x.is_cuda:
        raise _lib.KernelError(f"linear: the CUDA kernels take bf16 or fp16 activations, got {x.dtype}")
    return F.linear(x, weight, bias)
