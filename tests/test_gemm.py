"""tcgen05 GEMM vs a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DT = torch.bfloat16     # the 16-bit dtype under test; every test below runs once for bf16 and once for fp16


@pytest.fixture(autouse=True, params=[torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def _dtype(request):
    global DT
    DT = request.param
    yield
    DT = torch.bfloat16


def _ref(a, b, ta, tb):
    A = a.float().t() if ta else a.float()
    B = b.float() if tb else b.float().t()
    return A @ B


def _check(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < 2e-2, f"max err {err} vs scale {scale}"
    # bf16 output rounding dominates: mean relative error must be tiny
    rel = ((out.float() - ref).abs().mean() / (ref.abs().mean() + 1e-6)).item()
    assert rel < 8e-3, f"mean rel err {rel}"


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 264, 136), (1024, 128, 512),
                                    (384, 1000, 72), (4096, 4096, 1024)])
def test_gemm_layouts(ta, tb, M, N, K):
    from gpt_neox_b200.ops.gemm import gemm
    torch.manual_seed(0)
    if ta and M % 8:
        pytest.skip("transposed A needs M % 8 == 0")
    a = torch.randn((K, M) if ta else (M, K), device="cuda", dtype=DT)
    b = torch.randn((K, N) if tb else (N, K), device="cuda", dtype=DT)
    out = gemm(a, b, trans_a=ta, trans_b=tb)
    torch.cuda.synchronize()
    _check(out, _ref(a, b, ta, tb), K)


def test_gemm_epilogues():
    from gpt_neox_b200.ops.gemm import gemm
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device="cuda", dtype=DT)
    b = torch.randn(N, K, device="cuda", dtype=DT) * 0.05
    bias = torch.randn(N, device="cuda", dtype=DT)
    res = torch.randn(M, N, device="cuda", dtype=DT)
    pre = a.float() @ b.float().t() + bias.float()
    aux = torch.empty(M, N, device="cuda", dtype=DT)
    out = gemm(a, b, bias=bias, gelu="erf", aux_out=aux, residual=res)
    ref = torch.nn.functional.gelu(pre) + res.float()
    _check(aux, pre, K)
    _check(out, ref, K)
    out_t = gemm(a, b, bias=bias, gelu="tanh")
    _check(out_t, torch.nn.functional.gelu(pre, approximate="tanh"), K)
    # dgelu epilogue
    g = gemm(a, b, dgelu_aux=aux, dgelu="erf")
    x = aux.float().requires_grad_(True)
    torch.nn.functional.gelu(x).sum().backward()
    _check(g, (a.float() @ b.float().t()) * x.grad, K)
    # fp32 accumulate
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    gemm(a, b, out=acc, accumulate=True)
    gemm(a, b, out=acc, accumulate=True)
    _check(acc, 2 * (a.float() @ b.float().t()) + 1, K)


def test_linear_autograd():
    from gpt_neox_b200.ops.gemm import linear
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda", dtype=DT, requires_grad=True)
    w = (torch.randn(384, 256, device="cuda", dtype=DT) * 0.05).requires_grad_(True)
    b = torch.randn(384, device="cuda", dtype=DT).requires_grad_(True)
    y = linear(x, w, b)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(gy.float())
    _check(y, yr.detach(), 256)
    _check(x.grad, xr.grad, 384)
    _check(w.grad, wr.grad, 384)
    _check(b.grad, br.grad, 384)


def test_no_device_error():
    from gpt_neox_b200.ops import _lib
    assert _lib.read_device_error(clear=False) == 0
