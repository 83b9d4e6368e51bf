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


def test_fp8_model_loss_tracks_bf16_model():
    """Same weights, linear layers on fp8 tensor cores vs bf16: first losses agree, and the fp8 model trains."""
    from common import tiny_config
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.models.gpt2_model import cross_entropy
    base = dict(num_layers=2, hidden_size=256, num_attention_heads=4, seq_length=128, max_position_embeddings=128,
                synthetic_vocab_size=1000, attention_config=[[["flash"], 2]], distributed_backend="nccl",
                precision="bfloat16")
    models = []
    for fp8_on in (False, True):
        a = NeoXArgs.from_dict(tiny_config(**base, te_columnparallel=fp8_on, te_rowparallel=fp8_on))
        a.configure_distributed_args()
        a.build_tokenizer()
        mpu.destroy_model_parallel()
        initialize_megatron(a)
        models.append(training.get_model(a))
    models[1].load_state_dict(models[0].state_dict())
    torch.manual_seed(0)
    tok = torch.randint(0, 1000, (4, 129), device="cuda")
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    pos = torch.arange(128, device="cuda")[None].expand(4, -1)
    mask = torch.ones(4, 128, device="cuda")
    losses = []
    for m in models:
        l = cross_entropy(m((x, pos, None)), (y, mask))
        l.backward()
        losses.append(l.item())
    assert abs(losses[0] - losses[1]) < 0.05 * abs(losses[0]), losses
    g0 = dict(models[0].named_parameters())["sequential.2.mlp.linear1.weight"].grad.float()
    g1 = dict(models[1].named_parameters())["sequential.2.mlp.linear1.weight"].grad.float()
    assert ((g0 - g1).norm() / g0.norm()).item() < 0.2
    assert any(getattr(m, "fp8_meta", None) is not None for m in models[1].modules())
