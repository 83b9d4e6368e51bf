"""The allocation-free column-sum entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory at the moment they call in (a C/C++
runtime without PyTorch that has handed all HBM to its own arena, or a step running under a fixed
memory plan).  ``nx_colsum_bf16_noalloc`` serves them from a scratch array built into the library.
The test checks it against the regular entry point (which takes a caller workspace) on two calls in
a row: the second call reuses the scratch the first one left dirty.  It is collected last so that a
run stopping at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from gpt_neox_b200.ops import _lib
    fn = _lib.lib().nx_colsum_bf16_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_longlong, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    return fn


def _call(fn, x, out, accumulate=0):
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), x.shape[0], x.shape[1], x.stride(0),
              accumulate, stream)


def test_noalloc_matches_workspace_entry_point_twice():
    from gpt_neox_b200.ops.elementwise import colsum
    fn = _symbol()
    torch.manual_seed(0)
    torch.cuda.synchronize()
    for rows, n in [(4097, 520), (300, 4096)]:      # second call: different shape over the dirty scratch
        x = torch.randn(rows, n, device="cuda").to(torch.bfloat16)
        want = colsum(x, torch.float32)             # existing entry point, workspace from the caller
        got = torch.empty(n, device="cuda", dtype=torch.float32)
        assert _call(fn, x, got) == 0
        torch.cuda.synchronize()
        err = ((got - want).abs().max() / (want.abs().max() + 1e-6)).item()
        assert err < 1e-5, f"rows={rows} n={n}: relative error {err}"
        ref = x.float().sum(0)
        assert ((got - ref).abs().max() / (ref.abs().max() + 1e-6)).item() < 1e-5
    # accumulate adds into the output
    acc = got.clone()
    assert _call(fn, x, acc, accumulate=1) == 0
    torch.cuda.synchronize()
    assert ((acc - 2 * got).abs().max() / (got.abs().max() + 1e-6)).item() < 1e-5


@pytest.mark.parametrize("rows", [0, 5, 255, 1000])
def test_noalloc_few_rows_and_a_column_slice_with_a_wider_leading_dimension(rows):
    fn = _symbol()
    torch.manual_seed(1)
    full = torch.randn(rows, 1024, device="cuda").to(torch.bfloat16)
    x = full[:, 256:256 + 520]                       # ld = 1024 > N = 520, start 16-byte aligned
    got = torch.full((520,), 7.0, device="cuda", dtype=torch.float32)
    assert _call(fn, x, got) == 0
    torch.cuda.synchronize()
    ref = x.float().sum(0)
    assert (got - ref).abs().max().item() <= 1e-5 * (ref.abs().max().item() + 1.0)


def test_noalloc_on_a_side_stream():
    fn = _symbol()
    torch.manual_seed(2)
    x = torch.randn(2048, 768, device="cuda").to(torch.bfloat16)
    got = torch.empty(768, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        assert _call(fn, x, got) == 0
    side.synchronize()
    ref = x.float().sum(0)
    assert (got - ref).abs().max().item() <= 1e-5 * (ref.abs().max().item() + 1.0)


def test_noalloc_rejects_sizes_beyond_the_scratch():
    from gpt_neox_b200.ops import _lib
    fn = _symbol()
    x = torch.zeros(64 * 256, 16392, device="cuda", dtype=torch.bfloat16)    # 64 slabs x 16392 > 2^20
    out = torch.empty(16392, device="cuda", dtype=torch.float32)
    assert _call(fn, x, out) == 2                    # NX_ERR_ARG, nothing launched
    assert b"exceeds the built-in scratch" in _lib.lib().nx_last_error()
