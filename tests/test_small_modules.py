"""Small model pieces against their textbook statements: ALiBi slopes / bias, sinusoidal table, activation
selector (plain and gated), the FLOP model, and the Tee log writer."""
import math
import types

import pytest
import torch
import torch.nn.functional as F


def test_alibi_slopes_power_of_two_and_interpolated():
    from gpt_neox_b200.ops.attention import alibi_slopes
    s8 = alibi_slopes(8)
    torch.testing.assert_close(s8, torch.tensor([2.0 ** (-(i + 1)) for i in range(8)]))      # 2^(-8/n * (i+1)), n = 8
    s12 = alibi_slopes(12)                                                                  # 8 + 4 interpolated heads
    torch.testing.assert_close(s12[:8], s8)
    torch.testing.assert_close(s12[8:], torch.tensor([2.0 ** (-0.5 * (2 * i + 1)) for i in range(4)]))


def test_alibi_bias_is_minus_slope_times_distance_and_sliced_per_rank():
    from gpt_neox_b200.models.positional_embeddings import AliBi
    from gpt_neox_b200.ops.attention import alibi_slopes
    a = AliBi(8, mp_size=2, mp_rank=1)
    torch.testing.assert_close(a.slopes, alibi_slopes(8)[4:])
    x = torch.zeros(1, 4, 3, 5)                       # 3 queries at the end of 5 keys
    y = a(x)
    for h in range(4):
        for i in range(3):
            for j in range(5):
                qpos = i + 2
                want = -float(a.slopes[h]) * max(qpos - j, 0)
                assert float(y[0, h, i, j]) == pytest.approx(want)


def test_sinusoidal_table():
    from gpt_neox_b200.models.positional_embeddings import SinusoidalPositionalEmbedding
    e = SinusoidalPositionalEmbedding(8, precision=torch.float32)(torch.zeros(2, 5, 8))
    assert e.shape == (1, 5, 8)
    inv = [1.0 / 10000 ** (k / 8) for k in (0, 2, 4, 6)]
    for t in range(5):
        for k in range(4):
            assert float(e[0, t, k]) == pytest.approx(math.sin(t * inv[k]), abs=1e-6)
            assert float(e[0, t, 4 + k]) == pytest.approx(math.cos(t * inv[k]), abs=1e-6)


@pytest.mark.parametrize("name,ref", [
    ("gelu", F.gelu), ("relu", F.relu), ("silu", F.silu), ("swish", F.silu), ("softsign", F.softsign),
    ("mish", lambda x: x * torch.tanh(F.softplus(x)))])
def test_plain_activations(name, ref):
    from gpt_neox_b200.models.activations import get_activation
    a = types.SimpleNamespace(activation=name, onnx_safe=False, bias_gelu_fusion=False)
    fn, gated = get_activation(a)
    x, b = torch.randn(3, 8), torch.randn(8)
    assert not gated
    torch.testing.assert_close(fn(x), ref(x))
    torch.testing.assert_close(fn(x, b), ref(x + b))


def test_gelu_tanh_only_with_bias_gelu_fusion_and_gated_chunk_order():
    from gpt_neox_b200.models.activations import get_activation
    x = torch.randn(3, 8)
    fused, _ = get_activation(types.SimpleNamespace(activation="gelu", onnx_safe=False, bias_gelu_fusion=True))
    torch.testing.assert_close(fused(x), F.gelu(x, approximate="tanh"))
    for name, act in (("swiglu", F.silu), ("geglu", F.gelu), ("reglu", F.relu), ("glu", torch.sigmoid),
                      ("bilinear", lambda t: t)):
        fn, gated = get_activation(types.SimpleNamespace(activation=name, onnx_safe=False, bias_gelu_fusion=False))
        assert gated
        torch.testing.assert_close(fn(x), x[:, :4] * act(x[:, 4:]))      # first half value, second half gate
    with pytest.raises(ValueError):
        get_activation(types.SimpleNamespace(activation="nope", onnx_safe=False, bias_gelu_fusion=False))


def test_flops_model_matches_the_formula():
    from gpt_neox_b200.obs.logging import get_flops
    a = types.SimpleNamespace(padded_vocab_size=50304, train_batch_size=32, seq_length=2048, hidden_size=1024,
                              num_layers=12, checkpoint_activations=False, attention_config=["flash"] * 12,
                              num_attention_heads=16)
    want = 24 * 3 * 32 * 2048 * 12 * 1024 ** 2 * (1 + 2048 / (6 * 1024) + 50304 / (16 * 12 * 1024))
    assert get_flops(a, 2.0) == pytest.approx(want / 2.0)
    a.checkpoint_activations = True
    assert get_flops(a, 2.0) == pytest.approx(want / 2.0 * 4 / 3)               # recompute adds a forward
    assert get_flops(a, 2.0, use_checkpointing_factor=False) == pytest.approx(want / 2.0)


def test_tee_duplicates_writes(tmp_path, capsys):
    from gpt_neox_b200.obs.logging import Tee
    path = tmp_path / "log.txt"
    t = Tee(str(path), err=False)
    try:
        print("hello tee")
    finally:
        t.close() if hasattr(t, "close") else t.__del__()
    assert "hello tee" in path.read_text()
    assert "hello tee" in capsys.readouterr().out


def test_reference_helper_names_resolve_and_behave():
    import torch
    from megatron import mpu
    from megatron.checkpointing import get_checkpoint_name
    from megatron.model.fused_softmax import SoftmaxFusionTypes
    from megatron.model.utils import get_fusion_type
    from megatron.utils import get_total_params, is_bnb_available, make_viewless_tensor
    from types import SimpleNamespace as NS
    assert mpu.get_tensor_model_parallel_world_size() == mpu.get_model_parallel_world_size()
    assert mpu.get_tensor_model_parallel_rank() == mpu.get_model_parallel_rank()
    assert get_checkpoint_name("/ck", 12, mp_rank=3) == "/ck/iter_0000012/mp_rank_03/model_optim_rng.pt"
    assert get_checkpoint_name("/ck", 0, release=True, mp_rank=0).startswith("/ck/release/")
    assert get_fusion_type(NS(scaled_upper_triang_masked_softmax_fusion=True, scaled_masked_softmax_fusion=True)) \
        == SoftmaxFusionTypes.upper_triang
    assert get_fusion_type(NS(scaled_upper_triang_masked_softmax_fusion=False, scaled_masked_softmax_fusion=True)) \
        == SoftmaxFusionTypes.general
    assert get_fusion_type(NS(scaled_upper_triang_masked_softmax_fusion=False, scaled_masked_softmax_fusion=False)) \
        == SoftmaxFusionTypes.none
    assert isinstance(is_bnb_available(), bool)
    assert get_total_params(torch.nn.Linear(4, 3)) == 15
    base = torch.randn(4, 6, requires_grad=True)
    view = base.view(2, 12)
    out = make_viewless_tensor(view)
    assert view._base is not None and out._base is None and out.data_ptr() == view.data_ptr()
    out.sum().backward()
    assert torch.equal(base.grad, torch.ones_like(base))
    assert make_viewless_tensor(base) is base
    assert make_viewless_tensor(view.detach(), requires_grad=False, keep_graph=False)._base is None
