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


@pytest.mark.parametrize("recipe", ["delayed", "mxfp8"])
def test_fp8_model_loss_tracks_bf16_model(recipe):
    """Same weights, linear layers on fp8 tensor cores (per-tensor delayed scaling, or block scaling) vs bf16: first
    losses agree, and so do the weight gradients."""
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
        a = NeoXArgs.from_dict(tiny_config(**base, te_columnparallel=fp8_on, te_rowparallel=fp8_on,
                                           te_fp8_recipe=recipe))
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
    if recipe == "delayed":
        assert any(getattr(m, "fp8_meta", None) is not None for m in models[1].modules())
    else:
        from gpt_neox_b200.ops import fp8
        w = dict(models[1].named_parameters())["sequential.2.mlp.linear1.weight"]
        assert id(w) in fp8._MX_WEIGHTS                   # the block-scaled path ran (and cached its quantised weights)


# ------------------------------------------------------------------------------------------------ block-scaled (MXFP8)
@pytest.mark.parametrize("rows,cols,e5m2", [(300, 416, False), (128, 128, True), (5, 32, False), (1000, 4096, False)])
def test_mxfp8_quantiser_matches_the_pytorch_statement(rows, cols, e5m2):
    """One power-of-two scale per 32 elements of a row (the smallest that brings the group into range), values
    converted with saturation, scale bytes packed four to a word per 128-column block: bytes and words equal the
    PyTorch statement bit for bit."""
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(0)
    x = (torch.randn(rows, cols, device="cuda") * (torch.rand(rows, 1, device="cuda") * 40)).bfloat16()
    x[0, :32] = 0                                              # an all-zero group keeps scale 1
    x[-1, -32:] = 448.0 if not e5m2 else 57344.0               # exactly the format maximum: scale 1, no saturation
    q, sf = fp8.mxfp8_quantize(x, e5m2=e5m2)
    qr, sfr = fp8.mxfp8_quantize_reference(x, e5m2=e5m2)
    assert torch.equal(sf, sfr)
    assert torch.equal(q, qr)
    back = fp8.mxfp8_dequantize_reference(q, sf, e5m2=e5m2)
    tol = 2.0 ** -3 if e5m2 else 2.0 ** -4                      # half a unit of the last mantissa bit, relative
    assert ((back - x.float()).abs() <= tol * x.float().abs().reshape(rows, -1, 32).amax(-1, keepdim=True)
            .expand(rows, cols // 32, 32).reshape(rows, cols) + 1e-30).all()


def _sf_words(e):
    """exponents [rows, groups] -> scale words in the kernels' layout."""
    from gpt_neox_b200.ops import fp8
    rows, ngr = e.shape
    nkb = (ngr + 3) // 4
    pad = torch.full((rows, nkb * 4), 127, dtype=torch.int32, device=e.device)
    pad[:, :ngr] = e + 127
    by = torch.full((nkb, fp8._pad128(rows), 4), 127, dtype=torch.int32, device=e.device)
    by[:, :rows, :] = pad.reshape(rows, nkb, 4).permute(1, 0, 2)
    return (by[..., 0] | (by[..., 1] << 8) | (by[..., 2] << 16) | (by[..., 3] << 24)).to(torch.int32)


@pytest.mark.parametrize("pattern", ["unit", "a_rows", "a_kgroups", "b_rows", "b_kgroups", "random"])
def test_mxfp8_gemm_applies_every_scale_where_it_belongs(pattern):
    """Scale factors that vary only along one axis of one operand pin down the tensor-memory layout the kernel
    stages them in: each pattern must reproduce the fp32 product of the de-scaled operands."""
    from gpt_neox_b200.ops import _lib, fp8
    torch.manual_seed(2)
    M, N, K = 384, 256, 512
    a = torch.randn(M, K, device="cuda").clamp(-3, 3).to(torch.float8_e4m3fn)
    b = torch.randn(N, K, device="cuda").clamp(-3, 3).to(torch.float8_e4m3fn)
    g = K // 32
    ea = torch.zeros(M, g, dtype=torch.int32, device="cuda")
    eb = torch.zeros(N, g, dtype=torch.int32, device="cuda")
    rows = lambda n: (torch.arange(n, device="cuda", dtype=torch.int32) % 7 - 3).unsqueeze(1).expand(n, g).contiguous()   # noqa: E731
    kgr = lambda n: (torch.arange(g, device="cuda", dtype=torch.int32) % 5 - 2).unsqueeze(0).expand(n, g).contiguous()   # noqa: E731
    if pattern == "a_rows":
        ea = rows(M)
    elif pattern == "a_kgroups":
        ea = kgr(M)
    elif pattern == "b_rows":
        eb = rows(N)
    elif pattern == "b_kgroups":
        eb = kgr(N)
    elif pattern == "random":
        ea = torch.randint(-4, 5, (M, g), device="cuda", dtype=torch.int32)
        eb = torch.randint(-4, 5, (N, g), device="cuda", dtype=torch.int32)
    ref = (a.float().reshape(M, g, 32) * torch.exp2(ea.float()).unsqueeze(-1)).reshape(M, K) @ \
          (b.float().reshape(N, g, 32) * torch.exp2(eb.float()).unsqueeze(-1)).reshape(N, K).t()
    out = fp8.gemm_mxfp8(a.view(torch.uint8), _sf_words(ea), b.view(torch.uint8), _sf_words(eb))
    torch.cuda.synchronize()
    assert _lib.read_device_error() == 0
    torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=ref.abs().max().item() * 4e-3)


@pytest.mark.parametrize("tile", [0, 128, 192, 224, 256])
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (200, 136, 160), (1024, 768, 2048), (130, 8, 32)])
def test_mxfp8_gemm_matches_dequantised_matmul(M, N, K, tile):
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(3)
    a = (torch.randn(M, K, device="cuda") * (1 + 10 * torch.rand(M, 1, device="cuda"))).bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    a8, sa = fp8.mxfp8_quantize(a)
    b8, sb = fp8.mxfp8_quantize(b, e5m2=True)
    bias = torch.randn(N, device="cuda").bfloat16()
    got = fp8.gemm_mxfp8(a8, sa, b8, sb, b_e5m2=True, bias=bias, tile=tile)
    want = fp8.mxfp8_dequantize_reference(a8, sa) @ fp8.mxfp8_dequantize_reference(b8, sb, True).t() + bias.float()
    torch.testing.assert_close(got.float(), want, rtol=1e-2, atol=want.abs().max().item() * 4e-3)
    acc = torch.ones(M, N, device="cuda")
    fp8.gemm_mxfp8(a8, sa, b8, sb, b_e5m2=True, out=acc, accumulate=True, tile=tile)
    torch.testing.assert_close(acc, want - bias.float() + 1.0, rtol=1e-3, atol=want.abs().max().item() * 1e-4)
    # against the unquantised product: the error of block-scaled e4m3 x e5m2 operands
    exact = a.float() @ b.float().t()
    assert ((got.float() - bias.float() - exact).norm() / exact.norm()).item() < 0.08


def test_mxfp8_linear_tracks_16_bit_linear():
    """Forward, input gradient and weight gradient of the block-scaled linear against the fp32 statement."""
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(4)
    x = torch.randn(4, 96, 512, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(768, device="cuda").bfloat16().requires_grad_(True)
    y = fp8.mxfp8_linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    nerr = lambda u, v: ((u.float() - v).norm() / v.norm()).item()   # noqa: E731
    assert nerr(y, yr) < 0.06 and nerr(x.grad, xr.grad) < 0.12 and nerr(w.grad, wr.grad) < 0.12
    assert nerr(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("rows,cols,e5m2", [(64, 96, False), (320, 1024, True), (8192, 512, False)])
def test_mxfp8_dual_quantiser_gives_both_forms_from_one_read(rows, cols, e5m2):
    """The row-wise form equals the single quantiser's, the column-wise form equals quantising the transposed tensor."""
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(5)
    x = (torch.randn(rows, cols, device="cuda") * (torch.rand(rows, 1, device="cuda") * 30)).bfloat16()
    q, sf, qt, sft = fp8.mxfp8_quantize_dual(x, e5m2=e5m2)
    q1, sf1 = fp8.mxfp8_quantize_reference(x, e5m2=e5m2)
    q2, sf2 = fp8.mxfp8_quantize_reference(x.t().contiguous(), e5m2=e5m2)
    assert torch.equal(q, q1) and torch.equal(sf, sf1)
    assert torch.equal(qt, q2) and torch.equal(sft, sf2)


def test_mxfp8_weights_are_quantised_once_per_step():
    """The quantised forms of a weight are reused until the weight changes (a tensor version bump) or a new optimizer
    step is announced (the engine's fused update writes through raw pointers)."""
    from gpt_neox_b200.ops import fp8
    torch.manual_seed(6)
    x = torch.randn(64, 256, device="cuda").bfloat16()
    w = (torch.randn(128, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    fp8.mxfp8_linear(x, w)
    first = fp8._MX_WEIGHTS[id(w)][1][0]
    fp8.mxfp8_linear(x, w)
    assert fp8._MX_WEIGHTS[id(w)][1][0] is first
    with torch.no_grad():
        w.mul_(2.0)
    y = fp8.mxfp8_linear(x, w)
    assert fp8._MX_WEIGHTS[id(w)][1][0] is not first
    second = fp8._MX_WEIGHTS[id(w)][1][0]
    fp8.mxfp8_new_step()
    fp8.mxfp8_linear(x, w)
    assert fp8._MX_WEIGHTS[id(w)][1][0] is not second
    ref = x.float() @ w.detach().float().t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 0.06
