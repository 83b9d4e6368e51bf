"""Modules that carry the reference's fused-op and Transformer-Engine names (megatron/model/fused_softmax.py,
fused_bias_dropout.py, fused_rope.py, fused_layer_norm.py, transformer_engine.py), reached through the
``megatron`` import aliases and checked against plain PyTorch statements of each function."""
import math

import pytest
import torch


def test_fused_scale_mask_softmax_all_fusion_types():
    from megatron.model.fused_softmax import FusedScaleMaskSoftmax, SoftmaxFusionTypes
    torch.manual_seed(0)
    b, h, s = 2, 3, 16
    x = torch.randn(b, h, s, s)
    causal = torch.triu(torch.ones(s, s, dtype=torch.bool), 1).view(1, 1, s, s)
    mask_func = lambda scores, m: scores.masked_fill(m, -10000.0)
    ref = torch.softmax(mask_func(x * 0.5, causal), -1)
    for ft in SoftmaxFusionTypes:
        m = FusedScaleMaskSoftmax(False, False, ft, mask_func, True, 0.5)
        got = m(x, causal)
        assert torch.allclose(got, ref, atol=1e-6), ft
    m = FusedScaleMaskSoftmax(False, False, SoftmaxFusionTypes.general, mask_func, True, None)
    assert not m.is_kernel_available(None, b, h, s, s)
    assert torch.allclose(m(x, None), torch.softmax(x, -1), atol=1e-6)
    with pytest.raises(AssertionError):
        FusedScaleMaskSoftmax(False, True, SoftmaxFusionTypes.none, mask_func, False, 0.5)
    assert FusedScaleMaskSoftmax.get_batch_per_block(128, 128, 4, 8) >= 1


def test_bias_dropout_add_entry_points():
    from megatron.model.fused_bias_dropout import (bias_dropout_add_fused_inference, bias_dropout_add_fused_train,
                                                   get_bias_dropout_add)
    torch.manual_seed(0)
    x, bias, res = torch.randn(4, 2, 8), torch.randn(8), torch.randn(4, 2, 8)
    assert torch.allclose(bias_dropout_add_fused_inference(x, bias.expand_as(x), res, 0.3), x + bias + res)
    assert torch.allclose(get_bias_dropout_add(True)(x, bias.expand_as(x), res, 0.0), x + bias + res)
    out = bias_dropout_add_fused_train(x, bias.expand_as(x), res, 0.5)
    kept = (out - res).abs() > 0
    assert 0.2 < kept.float().mean() < 0.8
    assert torch.allclose((out - res)[kept], ((x + bias) * 2)[kept], atol=1e-5)


def test_fused_rope_entry_points_match_rotate_half():
    from megatron.model.fused_rope import fused_apply_rotary_pos_emb, fused_apply_rotary_pos_emb_cached
    torch.manual_seed(0)
    s, b, h, d, d2 = 8, 2, 3, 16, 8
    t = torch.randn(s, b, h, d)
    inv = 1.0 / (10000 ** (torch.arange(0, d2, 2).float() / d2))
    f = torch.outer(torch.arange(s).float(), inv)
    freqs = torch.cat([f, f], -1).view(s, 1, 1, d2)
    rot, rest = t[..., :d2], t[..., d2:]
    half = torch.cat([-rot[..., d2 // 2:], rot[..., :d2 // 2]], -1)
    ref = torch.cat([rot * freqs.cos() + half * freqs.sin(), rest], -1)
    assert torch.allclose(fused_apply_rotary_pos_emb(t, freqs), ref, atol=1e-5)
    out = fused_apply_rotary_pos_emb_cached(t, freqs.cos(), freqs.sin(), transpose_output_memory=True)
    assert torch.allclose(out, ref, atol=1e-5) and out.transpose(0, 1).is_contiguous()


def test_mixed_fused_norms_with_1p():
    from megatron.model.fused_layer_norm import MixedFusedLayerNorm, MixedFusedRMSNorm
    torch.manual_seed(0)
    x = torch.randn(5, 3, 32)
    ln = MixedFusedLayerNorm(32, eps=1e-5, apply_layernorm_1p=True, sequence_parallel=True)
    assert float(ln.weight.detach().abs().sum()) == 0 and ln.weight.sequence_parallel_grad_sync
    with torch.no_grad():
        ln.weight.normal_(0, 0.1)
        ln.bias.normal_(0, 0.1)
    ref = torch.nn.functional.layer_norm(x, (32,), ln.weight + 1, ln.bias, 1e-5)
    assert torch.allclose(ln(x), ref, atol=1e-5)
    rn = MixedFusedRMSNorm(32, eps=1e-6)
    with torch.no_grad():
        rn.scale.normal_(1, 0.1)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * rn.scale
    assert torch.allclose(rn(x), ref, atol=1e-5)
    qk = MixedFusedLayerNorm((4, 8))
    assert torch.allclose(qk(x.view(5, 3, 4, 8)), torch.nn.functional.layer_norm(x, (32,)).view(5, 3, 4, 8), atol=1e-5)


def test_transformer_engine_names_build_on_the_fp8_path():
    from common import tiny_config
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200.config import NeoXArgs
    from megatron.model.transformer_engine import (TEColumnParallelLinear, TEDelayedScaling, TELayerNorm,
                                                   TELayerNormMLP, TELinear, TERMSNorm, TERowParallelLinear)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(tiny_config(use_cpu_initialization=True, te_fp8_format="hybrid"))
    col = TEColumnParallelLinear(a, 64, 128, gather_output=False)
    row = TERowParallelLinear(a, 128, 64, input_is_parallel=True)
    assert col.use_fp8 and row.use_fp8 and not getattr(a, "te_columnparallel", False)     # the caller's args stay as given
    x = torch.randn(4, 2, 64)
    y, _ = col(x)
    z, _ = row(y)
    assert y.shape == (4, 2, 128) and z.shape == (4, 2, 64)                   # CPU: the fp32 oracle path runs
    assert TELinear(a, 64, 32)(x)[0].shape == (4, 2, 32)
    assert torch.allclose(TELayerNorm(64)(x), torch.nn.functional.layer_norm(x, (64,)), atol=1e-5)
    assert TERMSNorm(64)(x).shape == x.shape
    from gpt_neox_b200.models.init_functions import get_init_methods
    im, om = get_init_methods(a)
    out, bias = TELayerNormMLP(a, im, om)(x)
    assert out.shape == x.shape
    r = TEDelayedScaling(a)
    assert r.fp8_format == "hybrid" and r.amax_history_len == a.te_fp8_amax_history_len
    with r.fp8_context():
        pass
    a.te_fp8_format = "e5m2"
    with pytest.raises(ValueError):
        TEDelayedScaling(a)


def test_named_factories_and_functional_helpers():
    import io
    import numpy as np
    from megatron.data.indexed_dataset import read_longs, write_longs
    from megatron.model.activations import Gated_Activation, GeLUFunction, bias_gelu, bias_gelu_back, erf_gelu
    from megatron.model.fused_rope import FusedRoPECachedFunc
    from megatron.model.init_functions import (init_method_normal, scaled_init_method_normal, small_init_init_method,
                                               wang_init_method, xavier_normal_init_method)
    from megatron.model.moe_mlp import MemoryOptimizedParallelGroupedMLP, ParallelGroupedMLP
    from megatron.model.positional_embeddings import apply_rotary_pos_emb, rotate_half
    from megatron.model.rwkv import RUN_CUDA_RWKV
    torch.manual_seed(0)
    t = torch.empty(256, 256)
    assert abs(float(init_method_normal(0.02)(t).std()) - 0.02) < 2e-3
    assert abs(float(init_method_normal(0.02, use_mup_outer=True, mup_init_scale=3.0)(t).std()) - 0.06) < 6e-3
    assert abs(float(init_method_normal(0.02, mup_init_scale=3.0)(t, use_mup=True).std()) - 0.06) < 6e-3
    assert abs(float(scaled_init_method_normal(0.02, 8)(t).std()) - 0.02 / 4) < 1e-3
    assert abs(float(scaled_init_method_normal(0.02, 8, num_residuals_per_layer=1)(t).std()) - 0.02 / math.sqrt(8)) < 1e-3
    assert abs(float(small_init_init_method(256)(t).std()) - math.sqrt(2 / (5 * 256))) < 3e-3
    assert abs(float(wang_init_method(4, 256)(t).std()) - 2 / 4 / 16) < 3e-3
    assert xavier_normal_init_method()(t) is t
    x, b = torch.randn(5, 8), torch.randn(8)
    assert torch.allclose(erf_gelu(x), torch.nn.functional.gelu(x), atol=1e-6)
    assert torch.allclose(bias_gelu(b, x), torch.nn.functional.gelu(x + b, approximate="tanh"), atol=1e-5)
    assert torch.allclose(GeLUFunction.apply(x, b), bias_gelu(b, x))
    xr = x.clone().requires_grad_(True)
    torch.nn.functional.gelu(xr + b, approximate="tanh").sum().backward()
    assert torch.allclose(bias_gelu_back(torch.ones_like(x), b, x), xr.grad, atol=1e-5)
    g = Gated_Activation("swiglu")(torch.cat([x, x], -1))
    assert torch.allclose(g, x * torch.nn.functional.silu(x), atol=1e-6)
    assert torch.equal(rotate_half(torch.tensor([1., 2., 3., 4.])), torch.tensor([-3., -4., 1., 2.]))
    s, d = 6, 8
    q, k = torch.randn(s, 2, 3, d), torch.randn(s, 2, 3, d)
    inv = 1.0 / (10000 ** (torch.arange(0, d, 2).float() / d))
    f = torch.outer(torch.arange(s + 2).float(), inv)
    emb = torch.cat([f, f], -1)[:, None, None, :]
    q2, k2 = apply_rotary_pos_emb(q, k, emb.cos(), emb.sin(), offset=2)
    assert torch.allclose(q2, FusedRoPECachedFunc.apply(q, emb.cos()[2:], emb.sin()[2:]), atol=1e-5)
    assert (q2.norm(dim=-1) - q.norm(dim=-1)).abs().max() < 1e-4 and k2.shape == k.shape
    assert MemoryOptimizedParallelGroupedMLP is ParallelGroupedMLP
    B, T, H, N = 1, 5, 2, 4
    r, kk, v = (torch.randn(B, T, H * N) for _ in range(3))
    w, u = -torch.rand(B, T, H * N), torch.randn(H, N)
    from gpt_neox_b200.ops.wkv import wkv6_reference
    assert torch.allclose(RUN_CUDA_RWKV(B, T, H * N, H, r, kk, v, w, u), wkv6_reference(r, kk, v, w, u))
    buf = io.BytesIO()
    write_longs(buf, [1, 2, 2 ** 40])
    buf.seek(0)
    assert read_longs(buf, 3).tolist() == [1, 2, 2 ** 40]
    with pytest.raises(EOFError):
        read_longs(buf, 1)
