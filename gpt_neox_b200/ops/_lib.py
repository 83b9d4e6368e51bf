"""ctypes binding of ``lib/libneox_b200.so`` (the sm_100a kernel library).

The library is loaded lazily on first use.  On a machine with a CUDA device a missing
or unloadable library is a hard error: the CUDA ops never fall back silently to
PyTorch kernels.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB = None
_HALF = None
# NEOX_KERNEL_LIB=debug loads the range-checking build (python -m gpt_neox_b200.build --debug-bounds)
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / (
    "libneox_b200_dbg.so" if os.environ.get("NEOX_KERNEL_LIB") == "debug" else "libneox_b200.so")

c_void_p, c_int, c_ll, c_float = C.c_void_p, C.c_int, C.c_longlong, C.c_float


class KernelError(RuntimeError):
    """A native kernel launcher returned a non-zero status."""


class DeviceWaitTimeout(RuntimeError):
    """The device error word was set: a bounded wait inside a kernel ran out."""


#: the 16-bit floating-point dtypes the kernels are built for: every ``nx_*`` entry point that touches
#: 16-bit tensors exists twice, ``nx_name`` for bf16 and ``nx_name_f16`` for fp16 (same signature)
H16 = (torch.bfloat16, torch.float16)


def is_h16(t) -> bool:
    return t.dtype in H16


class _HalfView:
    """Attribute access on this object resolves ``nx_name`` to the fp16 build ``nx_name_f16`` where one
    exists (entry points without 16-bit tensors exist once and are shared)."""

    def __init__(self, lib):
        self._lib = lib

    def __getattr__(self, name):
        fn = getattr(self._lib, name + "_f16", None)
        if fn is None:
            fn = getattr(self._lib, name)
        setattr(self, name, fn)
        return fn


def _declare(lib):
    def sig(name, argtypes, restype=c_int):
        for nm in (name, name + "_f16"):
            try:
                fn = getattr(lib, nm)
            except AttributeError:
                continue
            fn.argtypes = argtypes
            fn.restype = restype

    P, I, L, F, U = c_void_p, c_int, c_ll, c_float, C.c_ulonglong
    sig("nx_last_error", [], C.c_char_p)
    sig("nx_read_device_error", [I])
    sig("nx_poison_device_error", [I])
    sig("nx_sm_count", [])
    sig("nx_set_wait_budget_cycles", [L])
    sig("nx_set_comm_jitter_ns", [I])
    sig("nx_comm_register_workspace", [U, L])
    sig("nx_comm_debug_bounds", [])
    sig("nx_mbar_timeout_probe", [P, P])
    sig("nx_wait_counter", [P, C.c_uint, P])
    sig("nx_abi_version", [])
    sig("nx_gemm_bf16", [P, P, P, I, I, I, L, L, L, I, I, P, P, P, P, L, I, F, P])
    sig("nx_gemm2_bf16", [P, P, P, I, I, I, L, L, L, I, I, P, P, P, P, L, I, F, P])
    sig("nx_norm_fwd", [I, P, P, P, P, P, P, P, P, P, L, I, F, P])
    sig("nx_norm_bwd_blocks", [L])
    sig("nx_norm_bwd", [I, P, P, P, P, P, P, P, P, P, P, P, P, P, P, L, I, I, P])
    sig("nx_bias_act_fwd", [P, P, P, L, I, I, P])
    sig("nx_bias_act_bwd", [P, P, P, P, L, I, I, P])
    sig("nx_gated_act_fwd", [P, P, L, I, I, P])
    sig("nx_gated_act_bwd", [P, P, P, L, I, I, P])
    sig("nx_bias_dropout_add", [P, P, P, P, P, L, I, F, U, U, P])
    sig("nx_dropout_bwd", [P, P, P, L, F, P])
    sig("nx_colsum_slabs", [L])
    sig("nx_colsum_bf16", [P, P, P, P, L, I, L, I, P])
    sig("nx_cast_f32_to_bf16", [P, P, L, F, P])
    sig("nx_softmax_causal_fwd", [P, P, L, I, I, F, P])
    sig("nx_softmax_masked_fwd", [P, P, P, I, I, I, I, I, F, P])
    sig("nx_softmax_bwd", [P, P, P, L, I, F, P])
    sig("nx_softmax_batch_per_block", [I, I, I, I])
    sig("nx_ce_fwd", [P, P, P, L, I, L, I, I, P])
    sig("nx_ce_bwd", [P, P, P, P, P, L, I, L, L, I, I, P])
    sig("nx_adamw_step", [P, P, P, P, P, L, F, F, F, F, F, F, F, I, P, P, I, P])
    sig("nx_adamw8bit_step", [P, P, P, P, P, P, P, L, F, F, F, F, F, F, F, I, P, P, I, P])
    sig("nx_sumsq", [P, L, P, I, P])
    sig("nx_clip_coef", [P, F, F, P, P, P])
    sig("nx_conv1d_silu_fwd", [P, L, L, P, P, P, L, L, I, I, I, I, P])
    sig("nx_conv1d_silu_bwd", [P, L, L, P, P, P, L, L, P, L, L, P, P, I, I, I, I, P])
    sig("nx_scan_chunks", [I])
    sig("nx_scan_channel_blocks", [I])
    sig("nx_selective_scan_fwd", [P, L, L, P, L, L, P, L, L, P, L, L, P, L, L, P, P, P, P, L, L, P, P, P, I, I, I, P])
    sig("nx_selective_scan_bwd", [P, L, L, P, L, L, P, L, L, P, L, L, P, L, L, P, P, P, P, L, L, P, P, P, L, L, P, P,
                                  P, P, P, P, P, I, I, I, P])
    sig("nx_wkv6_chunks", [I])
    sig("nx_wkv6_pass", [I, P, P, P, P, L, L, P, P, L, L, I, P, P, P, I, I, I, I, P])
    sig("nx_gemm_fp8", [P, P, P, I, I, I, L, L, L, I, I, P, P, I, I, P])
    sig("nx_fp8_quantize", [P, L, P, P, L, P, L, P, I, I, I, P])
    sig("nx_gemm_mxfp8", [P, P, P, I, I, I, L, L, L, P, P, L, L, I, I, P, P, I, I, I, P])
    sig("nx_mxfp8_quantize", [P, L, P, L, P, L, I, I, I, P])
    sig("nx_mxfp8_quantize_dual", [P, L, P, L, P, L, P, L, P, L, I, I, I, P])
    sig("nx_moe_blocks", [I])
    sig("nx_moe_max_rows", [I, I])
    sig("nx_moe_plan", [P, I, I, P, P, P, P, P, P, P, P])
    sig("nx_moe_gather_rows", [P, L, P, P, I, P, I, I, P])
    sig("nx_moe_combine", [P, P, P, I, P, I, I, P])
    sig("nx_moe_weight_grad", [P, P, P, I, P, I, I, P])
    sig("nx_gemm_bf16_grouped", [I, P, P, P, I, I, I, L, L, L, I, I, P, P, L, P, P, L, I, P])
    sig("nx_rope", [P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, I, I, P])
    sig("nx_embedding_fwd", [P, P, P, L, I, L, L, P])
    sig("nx_embedding_bwd", [P, P, P, L, I, L, L, P])
    sig("nx_flash_attn_fwd", [P] * 6 + [I] * 6 + [L] * 12 + [F, I, I, F, U, P, P, I, P])
    sig("nx_flash_attn_bwd", [P] * 11 + [I] * 6 + [L] * 24 + [F, I, I, F, U, P, P, I, P])
    return lib


def available() -> bool:
    return _LIB_PATH.exists()


def lib(like=None):
    """The kernel library.  ``like``: a tensor or dtype; for ``torch.float16`` the returned object resolves
    every entry point to its fp16 build."""
    global _LIB, _HALF
    if _LIB is not None:
        dt = getattr(like, "dtype", like)
        return _HALF if dt == torch.float16 else _LIB
    if _LIB is None:
        if not _LIB_PATH.exists():
            raise KernelError(
                f"{_LIB_PATH} is missing: build it with `python -m gpt_neox_b200.build` "
                "(the CUDA ops have no PyTorch fallback on a GPU)"
            )
        _LIB = _declare(C.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else 0))
        _HALF = _HalfView(_LIB)
    return lib(like)


def check(status: int, what: str = "kernel"):
    if status != 0:
        msg = lib().nx_last_error().decode(errors="replace")
        raise KernelError(f"{what} failed with status {status}: {msg}")


def ptr(t):
    """Device pointer of a tensor (or None) as a ctypes void pointer."""
    if t is None:
        return None
    if not t.is_cuda:
        # every kernel dereferences its pointers on the device: refuse a host tensor here instead
        # of letting the GPU fault on it
        raise KernelError(f"host tensor (shape {tuple(t.shape)}, {t.dtype}) passed to a CUDA kernel")
    return c_void_p(t.data_ptr())


def stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def read_device_error(clear: bool = True) -> int:
    return int(lib().nx_read_device_error(1 if clear else 0))


def set_wait_budget_cycles(cycles: int):
    """Cycle budget of every bounded wait (mbarrier / flag) in kernels launched afterwards on the current
    device; 0 restores the built-in default (4e9 cycles, about two seconds)."""
    check(lib().nx_set_wait_budget_cycles(int(cycles)), "nx_set_wait_budget_cycles")


def set_comm_jitter_ns(max_ns: int):
    """Debug aid: a pseudo-random sleep below ``max_ns`` nanoseconds in front of every cross-rank signal of the
    communication kernels launched afterwards on the current device (0 = off)."""
    check(lib().nx_set_comm_jitter_ns(int(max_ns)), "nx_set_comm_jitter_ns")


def register_workspace(base_ptr: int, nbytes: int):
    """Tell both kernel builds the size of a symmetric workspace (acted on by the range-checking debug build)."""
    lib().nx_comm_register_workspace(int(base_ptr), int(nbytes))
    lib(torch.float16).nx_comm_register_workspace(int(base_ptr), int(nbytes))


def raise_on_device_error():
    """Synchronising check of the device error word; raises DeviceWaitTimeout if set."""
    v = read_device_error(clear=True)
    if v != 0:
        raise DeviceWaitTimeout(f"device error word = 0x{v:x} (code {v & 0xff}, site {v >> 8})")
