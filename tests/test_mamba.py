"""Mamba: model-level CPU checks and kernel numerics against the fp32 PyTorch recurrences."""
import pytest
import torch

from common import run_distributed, tiny_config


def _train(rank, world, cfg, steps):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(2)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world, train_iters=steps, lr_decay_iters=steps))
    a.configure_distributed_args()
    a.build_tokenizer()
    losses = []
    training.collect_loss_for_unit_test = lambda l: losses.append(float(l))
    training.pretrain(a)
    return losses


def test_mamba_model_trains_on_cpu():
    cfg = tiny_config(attention_config=[[["mamba"], 2]], pos_emb="none", gpt_j_residual=False, norm="rmsnorm",
                      use_cpu_initialization=True, optimizer={"type": "Adam", "params": {"lr": 3e-3}})
    losses = run_distributed(_train, 1, cfg, 12)[0]
    assert all(l == l for l in losses)
    assert min(losses[6:]) < losses[0]


def test_mamba_tp2_sp_runs_on_cpu():
    cfg = tiny_config(attention_config=[[["mamba"], 2]], pos_emb="none", gpt_j_residual=False, norm="rmsnorm",
                      use_cpu_initialization=True, model_parallel_size=2, sequence_parallel=True)
    out = run_distributed(_train, 2, cfg, 3)
    assert out[0] == pytest.approx(out[1], rel=1e-6)


def test_conv_reference_is_causal():
    from gpt_neox_b200.ops.mamba import causal_conv1d_silu
    x = torch.randn(1, 10, 4)
    w, b = torch.randn(4, 4), torch.randn(4)
    y0 = causal_conv1d_silu(x, w, b)
    x2 = x.clone()
    x2[:, 6:] += 1.0
    y1 = causal_conv1d_silu(x2, w, b)
    assert torch.equal(y0[:, :6], y1[:, :6])


@pytest.mark.gpu
@pytest.mark.parametrize("L,D,W,bias", [(200, 192, 4, True), (64, 64, 3, False)])
def test_conv1d_silu_kernel(L, D, W, bias):
    from gpt_neox_b200.ops.mamba import causal_conv1d_silu, causal_conv1d_silu_reference
    torch.manual_seed(0)
    B = 3
    base = torch.randn(L, B, 2 * D, device="cuda", dtype=torch.bfloat16)
    x = base[..., :D].transpose(0, 1).detach().requires_grad_(True)      # strided [b, l, d] view
    w = (torch.randn(D, W, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    b = torch.randn(D, device="cuda").bfloat16().requires_grad_(True) if bias else None
    y = causal_conv1d_silu(x, w, b)
    g = torch.randn(B, L, D, device="cuda", dtype=torch.bfloat16)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if bias else None
    yr = causal_conv1d_silu_reference(xr, wr, br)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=3e-2, atol=0.15)
    if bias:
        torch.testing.assert_close(b.grad.float(), br.grad, rtol=3e-2, atol=0.15)


@pytest.mark.gpu
@pytest.mark.parametrize("L,D,use_z", [(300, 128, True), (128, 96, True), (40, 64, False)])
def test_selective_scan_kernel(L, D, use_z):
    from gpt_neox_b200.ops.mamba import selective_scan, selective_scan_reference
    torch.manual_seed(1)
    B, N = 2, 16
    dev = "cuda"
    mk = lambda *s: (torch.randn(*s, device=dev) * 0.5).bfloat16()
    x, dt, z = mk(B, L, D), mk(B, L, D), mk(B, L, D)
    bc = mk(L, B, 2 * N + 8)
    Bm, Cm = bc[..., 8:8 + N].transpose(0, 1), bc[..., 8 + N:].transpose(0, 1)    # strided views
    A = -(torch.rand(D, N, device=dev) * 4 + 0.5)
    Dp = torch.randn(D, device=dev)
    dtb = torch.randn(D, device=dev) * 0.5 - 2.0
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, dt, A, Bm, Cm, Dp, z, dtb)]
    ref = [t.detach().clone().float().requires_grad_(True) for t in (x, dt, A, Bm, Cm, Dp, z, dtb)]
    y = selective_scan(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], leaves[5],
                       leaves[6] if use_z else None, leaves[7])
    yr = selective_scan_reference(ref[0], ref[1], ref[2], ref[3], ref[4], ref[5], ref[6] if use_z else None, ref[7])
    g = torch.randn(B, L, D, device=dev).bfloat16()
    y.backward(g)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=3e-2, atol=3e-2)
    names = ["x", "dt", "A", "B", "C", "D", "z", "dt_bias"]
    for n, a, r in zip(names, leaves, ref):
        if n == "z" and not use_z:
            continue
        scale = r.grad.abs().max().item() + 1e-6
        err = (a.grad.float() - r.grad).abs().max().item()
        assert err <= 0.03 * scale + 1e-3, f"grad {n}: err {err} vs scale {scale}"
