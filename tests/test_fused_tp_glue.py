"""The autograd glue of the fused tensor-parallel linears (ops/fused_tp.py) on CPU, with a one-rank stand-in for the
symmetric-memory backend: gradients equal plain autograd, a pool slot is given back exactly once and before the fused
call that follows it, and every way of not getting a slot (no grad, input without gradient, pipeline parallelism, pool
exhausted) runs the copying form."""
import math

import pytest
import torch

from gpt_neox_b200.ops import fused_tp


def _gelu(x):
    return 0.5 * x * (1 + torch.erf(x / math.sqrt(2)))


def _dgelu(x):
    return 0.5 * (1 + torch.erf(x / math.sqrt(2))) + x * torch.exp(-0.5 * x * x) / math.sqrt(2 * math.pi)


class FakeBackend:
    """ws = 1: the gathered operand is the operand, the reduce-scatter is the identity."""
    ws = 1

    def __init__(self, slots):
        self.free, self.log = list(range(slots)), []

    def ag_gemm(self, x, w, *, trans_b=False, bias=None, gelu=None, aux_out=None, dgelu_aux=None, dgelu=None,
                aux_deriv=False, keep=None):
        pre = x.float() @ (w.float() if trans_b else w.float().t())
        if bias is not None:
            pre = pre + bias.float()
        if aux_out is not None:
            aux_out.copy_((_dgelu(pre) if aux_deriv else pre).to(aux_out.dtype))
        if dgelu_aux is not None:
            assert dgelu == "mul"
            pre = pre * dgelu_aux.float()
        y = (_gelu(pre) if gelu is not None else pre).to(x.dtype)
        self.log.append("ag_gemm")
        if keep is None:
            return y, x
        slot = self.free.pop(0) if (keep and self.free) else None
        return y, (x if slot is None else x.clone()), slot        # a pooled operand lives elsewhere than the ring

    def gemm_rs(self, a, w, *, trans_b=False, residual=None, bias=None, residual2=None, dgelu_aux=None, dgelu=None):
        y = a.float() @ (w.float() if trans_b else w.float().t())
        for t in (residual, bias, residual2):
            if t is not None:
                y = y + t.float()
        self.log.append("gemm_rs")
        return y.to(a.dtype)

    def pool_release(self, slot):
        assert slot not in self.free
        self.free.append(slot)
        self.log.append("release")


@pytest.fixture(autouse=True)
def _cpu_wgrad(monkeypatch):
    def wgrad(gy2, x2, weight):
        return (gy2.float().t() @ x2.float()).to(weight.dtype)
    monkeypatch.setattr(fused_tp, "wgrad", wgrad)


def _tensors(dtype=torch.float32):
    torch.manual_seed(0)
    x = torch.randn(12, 16, dtype=dtype)
    w1, b1 = torch.randn(24, 16, dtype=dtype) * 0.2, torch.randn(24, dtype=dtype) * 0.1
    w2 = torch.randn(16, 24, dtype=dtype) * 0.2
    return x, w1, b1, w2


@pytest.mark.parametrize("case", ["pooled", "pool_exhausted", "no_grad", "input_without_grad", "pipeline_parallel"])
def test_ag_linear_glue(case, monkeypatch):
    x, w, b, _ = _tensors()
    be = FakeBackend(0 if case == "pool_exhausted" else 2)
    if case == "pipeline_parallel":
        from gpt_neox_b200 import parallel as mpu
        monkeypatch.setattr(mpu, "get_pipe_parallel_world_size", lambda: 2)
    if case == "no_grad":
        with torch.no_grad():
            y = fused_tp.ag_linear(x, w, b, be)
        assert torch.allclose(y, x @ w.t() + b, atol=1e-5) and len(be.free) == 2 and "release" not in be.log
        return
    xp = x.clone().requires_grad_(case != "input_without_grad")
    wp, bp = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    y = fused_tp.ag_linear(xp, wp, bp, be)
    took = 2 - len(be.free) if case != "pool_exhausted" else 0
    assert took == (1 if case == "pooled" else 0)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = x.clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    (xr @ wr.t() + br).backward(g)
    assert torch.allclose(wp.grad, wr.grad, atol=1e-4) and torch.allclose(bp.grad, br.grad, atol=1e-4)
    if case != "input_without_grad":
        assert torch.allclose(xp.grad, xr.grad, atol=1e-4)
    if case == "pooled":
        assert len(be.free) == 2 and be.log.count("release") == 1
        assert be.log.index("release") < be.log.index("gemm_rs")          # given back before the fused call after it
    else:
        assert "release" not in be.log


@pytest.mark.parametrize("pooled", [True, False])
def test_mlp_gelu_sp_glue(pooled):
    x, w1, b1, w2 = _tensors()
    pf, bt, rs = torch.randn(12, 16) * 0.1, torch.randn(16) * 0.1, torch.randn(12, 16) * 0.1
    be = FakeBackend(1 if pooled else 0)
    leaves = [t.clone().requires_grad_(True) for t in (x, w1, b1, w2, pf, bt, rs)]
    out = fused_tp.mlp_gelu_sp(*leaves[:4], leaves[4], leaves[5], leaves[6], "erf", be)
    g = torch.randn_like(out)
    out.backward(g)
    ref = [t.clone().requires_grad_(True) for t in (x, w1, b1, w2, pf, bt, rs)]
    xr, w1r, b1r, w2r, pfr, btr, rsr = ref
    (_gelu(xr @ w1r.t() + b1r) @ w2r.t() + pfr + btr + rsr).backward(g)
    for a, r, name in zip(leaves, ref, ("x", "w1", "b1", "w2", "partial", "bias_total", "residual")):
        assert torch.allclose(a.grad, r.grad, atol=2e-4), name
    assert len(be.free) == (1 if pooled else 0)
    assert be.log.count("release") == (1 if pooled else 0)
    if pooled:
        assert be.log.index("release") < len(be.log) - 1 - be.log[::-1].index("gemm_rs")   # before the last fused call


@pytest.mark.parametrize("with_bias,with_res", [(True, True), (False, False)])
def test_linear_rs_glue(with_bias, with_res):
    x, _, _, w2 = _tensors()
    x = torch.randn(12, 24)
    b = torch.randn(16) * 0.1 if with_bias else None
    res = torch.randn(12, 16) * 0.1 if with_res else None
    be = FakeBackend(0)
    leaves = [t.clone().requires_grad_(True) if t is not None else None for t in (x, w2, b, res)]
    y = fused_tp.linear_rs(leaves[0], leaves[1], leaves[2], leaves[3], be)
    g = torch.randn_like(y)
    y.backward(g)
    ref = [t.clone().requires_grad_(True) if t is not None else None for t in (x, w2, b, res)]
    yr = ref[0] @ ref[1].t()
    if with_bias:
        yr = yr + ref[2]
    if with_res:
        yr = yr + ref[3]
    yr.backward(g)
    for a, r in zip(leaves, ref):
        if a is not None:
            assert torch.allclose(a.grad, r.grad, atol=2e-4)


def test_bias_gradient_goes_straight_into_main_grad_when_present():
    """With an fp32 ``main_grad`` on the bias (what the engine installs) the glue returns no gradient for it and the sum
    lands in ``main_grad``; on CPU the reduction kernel's stand-in adds it."""
    x, w, b, _ = _tensors()
    be = FakeBackend(1)
    xp, wp, bp = x.clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    bp.main_grad = torch.ones(b.shape, dtype=torch.float32)
    y = fused_tp.ag_linear(xp, wp, bp, be)
    g = torch.randn_like(y)
    y.backward(g)
    if bp.grad is None:                   # CUDA-only fast path is not taken on CPU tensors: the plain column sum is used
        assert torch.allclose(bp.main_grad, torch.ones_like(bp.main_grad) + g.sum(0), atol=1e-4)
    else:
        assert torch.allclose(bp.grad, g.sum(0), atol=1e-4)
