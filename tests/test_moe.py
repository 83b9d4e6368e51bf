"""Dropless MoE on one rank against a per-token loop (reference tests: tests/model/test_model_train.py moe params)."""
import pytest
import torch

from gpt_neox_b200 import parallel as mpu
from gpt_neox_b200.config import NeoXArgs
from gpt_neox_b200.models.init_functions import get_init_methods
from gpt_neox_b200.models.moe import ParallelDroplessMoE

from common import tiny_config


def _args(**kw):
    cfg = tiny_config(**{**dict(use_cpu_initialization=True, moe_num_experts=4, moe_top_k=2,
                             moe_expert_interval=1), **kw})
    a = NeoXArgs.from_dict(cfg)
    mpu.destroy_model_parallel()
    mpu.initialize_model_parallel(1)
    return a


@pytest.mark.parametrize("act,router", [("gelu", "topk"), ("swiglu", "topk"), ("gelu", "sinkhorn")])
def test_dropless_moe_matches_token_loop(act, router):
    a = _args(activation=act, moe_router_type=router, precision="fp32")
    torch.manual_seed(0)
    im, om = get_init_methods(a)
    moe = ParallelDroplessMoE(a, im, om).eval()
    x = torch.randn(8, 2, a.hidden_size, requires_grad=True)
    y = moe(x)
    assert y.shape == x.shape
    w, idx = moe.router(x)
    mlp = moe.experts.mlp
    E = a.moe_num_experts
    x2 = x.reshape(-1, a.hidden_size)
    want = torch.zeros_like(x2)
    for t in range(x2.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            w1 = mlp.w1.view(E, -1, a.hidden_size)[e]
            w2 = mlp.w2.view(E, -1, a.hidden_size)[e]
            if act == "swiglu":
                w3 = mlp.w3.view(E, -1, a.hidden_size)[e]
                h = torch.nn.functional.silu(x2[t] @ w1.T) * (x2[t] @ w3.T)
            else:
                h = torch.nn.functional.gelu(x2[t] @ w1.T)
            want[t] += w[t, j] * (h @ w2)
    torch.testing.assert_close(y.reshape(-1, a.hidden_size), want, rtol=1e-4, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    assert mlp.w1.grad is not None and moe.router.layer.weight.grad is not None


def test_sinkhorn_training_balances_and_is_differentiable():
    a = _args(moe_router_type="sinkhorn", precision="fp32", moe_top_k=1)
    im, om = get_init_methods(a)
    moe = ParallelDroplessMoE(a, im, om).train()
    x = torch.randn(16, 2, a.hidden_size, requires_grad=True)
    moe(x).sum().backward()
    assert torch.isfinite(x.grad).all()
