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


@pytest.mark.gpu
@pytest.mark.parametrize("T,k,E,h,ffn", [(512, 2, 4, 256, 512), (300, 1, 8, 128, 256), (1024, 2, 8, 768, 3072)])
def test_moe_kernel_path_matches_torch_path(T, k, E, h, ffn):
    """Plan / permute / grouped-GEMM kernels against the per-expert torch loop with the same weights."""
    from gpt_neox_b200.ops import _lib
    from gpt_neox_b200.ops import moe as M
    torch.manual_seed(0)
    dev = "cuda"
    x = torch.randn(T, h, device=dev).bfloat16().requires_grad_(True)
    w1 = (torch.randn(E * ffn, h, device=dev) * 0.05).bfloat16().requires_grad_(True)
    w2 = (torch.randn(E * ffn, h, device=dev) * 0.05).bfloat16().requires_grad_(True)
    logits = torch.randn(T, E, device=dev)
    wts, idx = torch.softmax(logits, -1).topk(k, dim=-1)
    wts = wts.bfloat16().requires_grad_(True)
    plan = M.Plan(idx, E)
    counts = torch.bincount(idx.reshape(-1), minlength=E)
    assert torch.equal(plan.counts.long(), counts)
    off = plan.offsets.long()
    assert bool((off % 128 == 0).all()) and bool(((off[1:] - off[:-1]) >= counts).all())
    # stable: copies of one expert keep their original order
    d = plan.dest_row.long()
    for e in range(E):
        rows = d[idx.reshape(-1) == e]
        assert bool((rows[1:] > rows[:-1]).all()) and (len(rows) == 0 or int(rows[0]) == int(off[e]))
    out = M.experts_gelu(x, wts, idx, w1, w2, E)
    g = torch.randn_like(out)
    out.backward(g)
    # fp32 statement
    xr, w1r, w2r, wr = (t.detach().float().requires_grad_(True) for t in (x, w1, w2, wts))
    ref = torch.zeros(T, h, device=dev)
    for e in range(E):
        sel = (idx == e)
        tok, slot = sel.nonzero(as_tuple=True)
        if len(tok) == 0:
            continue
        hh = torch.nn.functional.gelu(xr[tok] @ w1r[e * ffn:(e + 1) * ffn].t())
        ref = ref.index_add(0, tok, (hh @ w2r[e * ffn:(e + 1) * ffn]) * wr[tok, slot].unsqueeze(-1))
    ref.backward(g.float())
    rel = lambda a, b: ((a.float() - b).norm() / (b.norm() + 1e-9)).item()
    assert rel(out, ref) < 2e-2
    assert rel(x.grad, xr.grad) < 3e-2 and rel(w1.grad, w1r.grad) < 3e-2 and rel(w2.grad, w2r.grad) < 3e-2
    assert rel(wts.grad, wr.grad) < 3e-2
    assert _lib.read_device_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("ws,T,k,E,h,ffn", [(2, 200, 2, 4, 256, 512), (4, 96, 1, 8, 128, 256), (8, 64, 2, 8, 768, 1024)])
def test_expert_parallel_peer_memory_path_matches_fp32_oracle(ws, T, k, E, h, ffn):
    """Expert parallelism over peer memory with the ranks emulated on one GPU: ``ws`` workspaces driven in
    lockstep phase by phase (stream order stands in for the rank barriers), against the fp32 per-expert loop
    over all ranks' tokens.  Covers the pull-gather, the pull-combine and the routing-weight gradient."""
    from gpt_neox_b200.ops import _lib
    from gpt_neox_b200.ops import moe_ep as EP
    torch.manual_seed(1)
    dev = "cuda"
    El = E // ws
    w1 = (torch.randn(E * ffn, h, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(E * ffn, h, device=dev) * 0.05).bfloat16()
    xs = [torch.randn(T, h, device=dev).bfloat16() for _ in range(ws)]
    routed = [torch.softmax(torch.randn(T, E, device=dev), -1).topk(k, dim=-1) for _ in range(ws)]
    wts = [r[0].bfloat16() for r in routed]
    idx = [r[1] for r in routed]
    gs = [torch.randn(T, h, device=dev).bfloat16() for _ in range(ws)]
    w1s = [w1[r * El * ffn:(r + 1) * El * ffn].contiguous() for r in range(ws)]
    w2s = [w2[r * El * ffn:(r + 1) * El * ffn].contiguous() for r in range(ws)]
    Ws = EP.EpWorkspace.emulated(ws, T, k, h, El)
    ids = [i.reshape(-1).to(torch.int32) for i in idx]
    wfs = [w.reshape(-1).contiguous() for w in wts]
    for r in range(ws):
        EP.fwd_publish(Ws[r], xs[r], ids[r])
    st = [EP.fwd_experts(Ws[r], w1s[r], w2s[r], "erf") for r in range(ws)]
    outs = [EP.fwd_combine(Ws[r], ids[r], wfs[r]) for r in range(ws)]
    for r in range(ws):
        EP.bwd_publish(Ws[r], gs[r], wfs[r])
    dws = [EP.bwd_experts(Ws[r], *st[r], w1s[r], w2s[r], "erf") for r in range(ws)]
    back = [EP.bwd_combine(Ws[r], ids[r]) for r in range(ws)]
    # fp32 statement over the concatenated tokens
    X = torch.cat(xs).float().requires_grad_(True)
    Wt = torch.cat(wts).float().requires_grad_(True)
    I = torch.cat(idx)
    w1r, w2r = w1.float().requires_grad_(True), w2.float().requires_grad_(True)
    ref = torch.zeros(ws * T, h, device=dev)
    for e in range(E):
        tok, slot = (I == e).nonzero(as_tuple=True)
        if len(tok) == 0:
            continue
        hh = torch.nn.functional.gelu(X[tok] @ w1r[e * ffn:(e + 1) * ffn].t())
        ref = ref.index_add(0, tok, (hh @ w2r[e * ffn:(e + 1) * ffn]) * Wt[tok, slot].unsqueeze(-1))
    ref.backward(torch.cat(gs).float())
    rel = lambda a, b: ((a.float() - b).norm() / (b.norm() + 1e-9)).item()
    assert rel(torch.cat(outs), ref) < 2e-2
    assert rel(torch.cat([b[0] for b in back]), X.grad) < 3e-2
    assert rel(torch.cat([b[1].view(T, k) for b in back]), Wt.grad) < 3e-2
    assert rel(torch.cat([d[0] for d in dws]), w1r.grad) < 3e-2
    assert rel(torch.cat([d[1] for d in dws]), w2r.grad) < 3e-2
    assert _lib.read_device_error() == 0
