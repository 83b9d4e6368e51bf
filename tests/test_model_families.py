"""RWKV-6, gMLP / aMLP and mixed stacks build and train through the public training entry on CPU;
kernel numerics of the WKV recurrence on the GPU."""
import pytest
import torch

from common import run_distributed, tiny_config
from test_mamba import _train


@pytest.mark.parametrize("name,over", [
    ("rwkv", dict(attention_config=[[["rwkv"], 2]], pos_emb="none", gpt_j_residual=False, hidden_size=64,
                  num_attention_heads=2)),
    ("gmlp", dict(attention_config=[[["gmlp"], 2]], pos_emb="none", gpt_j_residual=False)),
    ("amlp", dict(attention_config=[[["amlp"], 2]], pos_emb="none", gpt_j_residual=False, gmlp_attn_dim=16)),
    ("mixed", dict(attention_config=[[["global"], 1], [["mamba"], 1]], num_layers=2, gpt_j_residual=False)),
])
def test_family_trains_on_cpu(name, over):
    cfg = tiny_config(**{**dict(use_cpu_initialization=True), **over})
    losses = run_distributed(_train, 1, cfg, 6)[0]
    assert all(l == l and l < 20 for l in losses), losses


def test_wkv_decay_gradient_identity():
    """dL/dw obtained from gr and gk by the reverse cumulative sum equals autograd's."""
    from gpt_neox_b200.ops.wkv import decay_grad_from_gr_gk, wkv6_reference
    torch.manual_seed(0)
    B, T, H, N = 2, 10, 2, 8
    C = H * N
    r, k, v = (torch.randn(B, T, C, requires_grad=True) for _ in range(3))
    w = (torch.randn(B, T, C) - 1).requires_grad_(True)
    u = torch.randn(H, N, requires_grad=True)
    y = wkv6_reference(r, k, v, w, u)
    gy = torch.randn_like(y)
    gr, gk, gv, gw, gu = torch.autograd.grad(y, (r, k, v, w, u), gy)
    gw2, gu2 = decay_grad_from_gr_gk(r.detach(), k.detach(), v.detach(), w.detach(), u.detach(), gy, gr, gk)
    torch.testing.assert_close(gw2, gw, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(gu2, gu, rtol=1e-3, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("T,H,N", [(300, 3, 64), (128, 2, 32), (50, 1, 64)])
def test_wkv6_kernel(T, H, N):
    from gpt_neox_b200.ops.wkv import wkv6, wkv6_reference
    torch.manual_seed(2)
    B, C, dev = 2, H * N, "cuda"
    mk = lambda: (torch.randn(T, B, C, device=dev) * 0.5).bfloat16().transpose(0, 1)
    r, k, v = mk(), mk(), mk()
    w = (torch.randn(T, B, C, device=dev) * 0.5 - 1.5).bfloat16().transpose(0, 1)
    u = (torch.randn(H, N, device=dev) * 0.3).bfloat16()
    leaves = [t.detach().clone().requires_grad_(True) for t in (r, k, v, w, u)]
    ref = [t.detach().float().clone().requires_grad_(True) for t in (r, k, v, w, u)]
    y = wkv6(*leaves)
    yr = wkv6_reference(*ref)
    gy = (torch.randn(B, T, C, device=dev) * 0.5).bfloat16()
    y.backward(gy)
    yr.backward(gy.float())
    scale = yr.abs().max().item()
    assert (y.float() - yr).abs().max().item() <= 0.02 * scale + 1e-2
    for n, a, b in zip("rkvwu", leaves, ref):
        s = b.grad.abs().max().item() + 1e-6
        err = (a.grad.float() - b.grad).abs().max().item()
        assert err <= 0.04 * s + 1e-2, f"grad {n}: err {err} scale {s}"


def test_sparse_layouts_are_causal_and_have_their_patterns():
    from gpt_neox_b200.models.sparse_attention import block_layout, token_mask
    nb = 16
    fixed = block_layout("sparse_fixed", nb, {"num_local_blocks": 4, "num_global_blocks": 1})
    assert fixed[5, 4] and fixed[5, 7] and not fixed[5, 8 + 1]          # dense inside window [4, 8)
    assert fixed[9, 3] and fixed[15, 7] and not fixed[9, 2]               # window summaries (last block) are global
    local = block_layout("local", nb, {"num_sliding_window_blocks": 4})
    assert local[6, 4] and local[6, 6] and not local[6, 3] and not local[6, 7]
    bb = block_layout("bigbird", nb, {})
    assert bb[10, 0] and bb[0, 10] and bb[10, 9] and bb[10, 11]
    m = token_mask("bslongformer", 100, {"block": 16})
    assert m.shape == (1, 1, 100, 100)
    allowed = ~m[0, 0]
    assert not torch.triu(allowed, 1).any()                               # causal
    assert allowed.diagonal().all() and allowed[:, 0].all()               # self and the global first block


@pytest.mark.parametrize("kind", ["local", "sparse_fixed", "sparse_variable", "bigbird", "bslongformer"])
def test_sparse_attention_types_train_on_cpu(kind):
    cfg = tiny_config(use_cpu_initialization=True, attention_config=[[[kind], 2]], sparsity_config={"block": 4})
    losses = run_distributed(_train, 1, cfg, 3)[0]
    assert all(l == l for l in losses)
