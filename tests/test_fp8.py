"""FP8 GEMM / quantisation kernels against fp32 PyTorch statements of the same quantised computation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,e5m2", [(256, 512, False), (200, 328, True), (64, 64, False)])
def test_quantize_matches_torch_cast(rows, cols, e5m2):
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(0)
    x = (torch.randn(rows, cols, device="cuda") * 3).bfloat16()
    meta = fp8.Fp8TensorMeta("cuda", e5m2=e5m2)
    meta.scale.fill_(8.0)
    q, qt = fp8.quantize(x, meta, transpose=True)
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    want = (x.float() * 8.0).clamp(-meta.fp8_max, meta.fp8_max).to(dt)
    assert torch.equal(q.view(dt).float(), want.float())
    assert torch.equal(qt, q.t().contiguous())
    assert meta.amax.item() == pytest.approx(x.float().abs().max().item())


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1024, 768, 1024), (136, 264, 144)])
def test_fp8_gemm_matches_dequantised_matmul(M, N, K):
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ma, mb = fp8.Fp8TensorMeta("cuda"), fp8.Fp8TensorMeta("cuda", e5m2=True)
    ma.scale.fill_(16.0), mb.scale.fill_(4.0)
    a8, _ = fp8.quantize(a, ma)
    b8, _ = fp8.quantize(b, mb)
    alpha = 1.0 / (ma.scale * mb.scale)
    bias = torch.randn(N, device="cuda").bfloat16()
    got = fp8.gemm_fp8(a8, b8, alpha, b_e5m2=True, bias=bias)
    want = fp8.dequantize_reference(a8, 16.0) @ fp8.dequantize_reference(b8, 4.0, True).t() + bias.float()
    torch.testing.assert_close(got.float(), want, rtol=1e-2, atol=5e-2)
    acc = torch.ones(M, N, device="cuda")
    fp8.gemm_fp8(a8, b8, alpha, b_e5m2=True, out=acc, accumulate=True)
    torch.testing.assert_close(acc, want - bias.float() + 1.0, rtol=1e-3, atol=1e-2)
    from gpt_neox_b200.ops import _lib
    assert _lib.read_device_error() == 0


def test_fp8_linear_tracks_bf16_linear():
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(2)
    x = torch.randn(4, 64, 256, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(512, device="cuda").bfloat16().requires_grad_(True)
    meta = fp8.Fp8LinearMeta("cuda")
    g = torch.randn(4, 64, 512, device="cuda").bfloat16()
    for _ in range(3):                       # first pass runs with unit scales; later passes use the history
        x.grad = w.grad = b.grad = None
        y = fp8.fp8_linear(x, w, b, meta)
        y.backward(g)
        meta.roll()
    yr = torch.nn.functional.linear(x.float(), w.float(), b.float())
    gx, gw, gb = torch.autograd.grad(yr, (x, w, b), g.float())
    rel = lambda a, r: ((a.float() - r).norm() / r.norm()).item()
    assert rel(y, yr) < 0.06 and rel(x.grad, gx) < 0.1 and rel(w.grad, gw) < 0.1 and rel(b.grad, gb) < 0.02
    assert meta.x.scale.item() > 1.0
