"""Every memory-bound / fused CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = torch.bfloat16     # the 16-bit dtype under test; every test below runs once for bf16 and once for fp16


@pytest.fixture(autouse=True, params=[torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def _dtype(request):
    global DT
    DT = request.param
    yield
    DT = torch.bfloat16


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()


def bf(*shape, scale=1.0, grad=False):
    t = (torch.randn(*shape, device=DEV) * scale).to(DT)
    return t.requires_grad_(grad)


@pytest.mark.parametrize("rows,H", [(7, 64), (300, 512), (1024, 2048), (33, 4096), (5, 6144), (700, 8192),
                                     (40, 16384), (20000, 1024), (5001, 6144)])   # the last two wrap the stage ring
def test_layernorm_fwd_bwd(rows, H):
    from gpt_neox_b200.ops.norm import layer_norm
    torch.manual_seed(0)
    x, w, b = bf(rows, H, grad=True), (1 + 0.1 * torch.randn(H, device=DEV)).to(DT).requires_grad_(True), \
        bf(H, scale=0.1, grad=True)
    y = layer_norm(x, w, b, 1e-5)
    g = bf(rows, H)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = F.layer_norm(xr, (H,), wr, br, 1e-5)
    yr.backward(g.float())
    assert rel(y, yr) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    assert rel(w.grad, wr.grad) < 2e-2
    assert rel(b.grad, br.grad) < 2e-2


def test_dual_layernorm_matches_two_norms():
    from gpt_neox_b200.ops.norm import dual_layer_norm
    torch.manual_seed(1)
    rows, H = 257, 1024
    x = bf(rows, H, grad=True)
    ws = [(1 + 0.1 * torch.randn(H, device=DEV)).to(DT).requires_grad_(True) for _ in range(2)]
    bs = [bf(H, scale=0.1, grad=True) for _ in range(2)]
    y1, y2 = dual_layer_norm(x, ws[0], bs[0], ws[1], bs[1], 1e-5)
    g1, g2 = bf(rows, H), bf(rows, H)
    (y1 * g1).sum().backward(retain_graph=True)
    (y2 * g2).sum().backward()
    xr = x.detach().float().requires_grad_(True)
    wr = [w.detach().float().requires_grad_(True) for w in ws]
    br = [b.detach().float().requires_grad_(True) for b in bs]
    r1 = F.layer_norm(xr, (H,), wr[0], br[0], 1e-5)
    r2 = F.layer_norm(xr, (H,), wr[1], br[1], 1e-5)
    ((r1 * g1.float()).sum() + (r2 * g2.float()).sum()).backward()
    assert rel(y1, r1) < 1e-2 and rel(y2, r2) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    for i in range(2):
        assert rel(ws[i].grad, wr[i].grad) < 2e-2
        assert rel(bs[i].grad, br[i].grad) < 2e-2


@pytest.mark.parametrize("rows,H", [(1000, 4096), (77, 6144), (300, 8192), (9, 16384), (5, 32768), (9000, 4096)])
def test_dual_layernorm_with_residual_carry_one_backward_pass(rows, H):
    """(x, y1, y2) = dual norm with the residual stream carried through the node: dx = g_res + both
    norm gradients from ONE backward kernel launch."""
    from gpt_neox_b200.ops.norm import dual_layer_norm
    torch.manual_seed(4)
    x = bf(rows, H, grad=True)
    ws = [(1 + 0.1 * torch.randn(H, device=DEV)).to(DT).requires_grad_(True) for _ in range(2)]
    bs = [bf(H, scale=0.1, grad=True) for _ in range(2)]
    res, y1, y2 = dual_layer_norm(x, ws[0], bs[0], ws[1], bs[1], 1e-5, carry=True)
    g0, g1, g2 = bf(rows, H), bf(rows, H), bf(rows, H)
    ((res * g0).sum() + (y1 * g1).sum() + (y2 * g2).sum()).backward()
    xr = x.detach().float().requires_grad_(True)
    wr = [w.detach().float().requires_grad_(True) for w in ws]
    br = [b.detach().float().requires_grad_(True) for b in bs]
    r1 = F.layer_norm(xr, (H,), wr[0], br[0], 1e-5)
    r2 = F.layer_norm(xr, (H,), wr[1], br[1], 1e-5)
    ((xr * g0.float()).sum() + (r1 * g1.float()).sum() + (r2 * g2.float()).sum()).backward()
    assert torch.equal(res, x)
    assert rel(y1, r1) < 1e-2 and rel(y2, r2) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    for i in range(2):
        assert rel(ws[i].grad, wr[i].grad) < 2e-2
        assert rel(bs[i].grad, br[i].grad) < 2e-2


def test_rmsnorm_carry_adds_residual_gradient():
    from gpt_neox_b200.ops.norm import rms_norm
    torch.manual_seed(5)
    rows, H = 300, 4096
    x, w = bf(rows, H, grad=True), (1 + 0.1 * torch.randn(H, device=DEV)).to(DT).requires_grad_(True)
    res, y = rms_norm(x, w, 1e-6, carry=True)
    g0, g = bf(rows, H), bf(rows, H)
    ((res * g0).sum() + (y * g).sum()).backward()
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = wr * (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6))
    ((xr * g0.float()).sum() + (yr * g.float()).sum()).backward()
    assert rel(x.grad, xr.grad) < 2e-2
    assert rel(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("rows,H", [(64, 256), (513, 4096), (12000, 2048)])
def test_rmsnorm_fwd_bwd(rows, H):
    from gpt_neox_b200.ops.norm import rms_norm
    torch.manual_seed(2)
    x, w = bf(rows, H, grad=True), (1 + 0.1 * torch.randn(H, device=DEV)).to(DT).requires_grad_(True)
    y = rms_norm(x, w, 1e-8)
    g = bf(rows, H)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = wr * (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-8))
    yr.backward(g.float())
    assert rel(y, yr) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    assert rel(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("act", ["gelu", "gelu_tanh", "relu", "silu"])
def test_bias_act(act):
    from gpt_neox_b200.ops.elementwise import _torch_act, bias_act
    torch.manual_seed(3)
    x, b = bf(100, 768, grad=True), bf(768, grad=True)
    y = bias_act(x, b, act)
    g = bf(100, 768)
    y.backward(g)
    xr, br = x.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    yr = _torch_act(act, xr + br)
    yr.backward(g.float())
    assert rel(y, yr) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    assert rel(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("kind", ["swiglu", "geglu", "reglu", "bilinear", "glu"])
def test_gated_act(kind):
    from gpt_neox_b200.ops.elementwise import GATED, _torch_act, gated_act
    torch.manual_seed(4)
    x = bf(77, 512, grad=True)
    y = gated_act(x, kind)
    g = bf(77, 256)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    v, gate = xr.chunk(2, dim=-1)
    yr = v * _torch_act(GATED[kind], gate)
    yr.backward(g.float())
    assert rel(y, yr) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2


def test_bias_dropout_add_and_colsum():
    from gpt_neox_b200.ops.elementwise import bias_dropout_add, colsum
    torch.manual_seed(5)
    x, b, r = bf(64, 1024, grad=True), bf(1024, grad=True), bf(64, 1024, grad=True)
    y = bias_dropout_add(x, b, r, 0.0, True)
    assert rel(y, x.float() + b.float() + r.float()) < 1e-2
    y.sum().backward()
    assert rel(b.grad, torch.full((1024,), 64.0, device=DEV)) < 1e-2
    # dropout: kept fraction and scaling
    x2 = torch.ones(512, 1024, device=DEV, dtype=DT, requires_grad=True)
    y2 = bias_dropout_add(x2, None, None, 0.25, True)
    kept = (y2 != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.02
    assert abs(y2.max().item() - 1 / 0.75) < 0.02
    y2.sum().backward()
    assert torch.equal((x2.grad != 0), (y2 != 0))
    big = bf(4097, 520)
    assert rel(colsum(big, torch.float32), big.float().sum(0)) < 1e-2


def test_softmax_causal_and_masked():
    from gpt_neox_b200.ops.softmax import scaled_causal_softmax, scaled_masked_softmax
    torch.manual_seed(6)
    x = bf(6, 200, 200, grad=True)
    y = scaled_causal_softmax(x, 0.37)
    g = bf(6, 200, 200)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    keep = torch.ones(200, 200, dtype=torch.bool, device=DEV).tril()
    yr = torch.softmax((xr * 0.37).masked_fill(~keep, float("-inf")), -1)
    yr.backward(g.float())
    assert rel(y, yr) < 1e-2
    assert rel(x.grad, xr.grad) < 3e-2
    x4 = bf(2, 3, 50, 3000, grad=True)          # longer than the reference kernels' 2048 cap
    mask = torch.rand(2, 1, 50, 3000, device=DEV) < 0.3
    y4 = scaled_masked_softmax(x4, mask, 0.5)
    g4 = bf(2, 3, 50, 3000)
    y4.backward(g4)
    x4r = x4.detach().float().requires_grad_(True)
    y4r = torch.softmax((x4r * 0.5).masked_fill(mask, -10000.0), -1)
    y4r.backward(g4.float())
    assert rel(y4, y4r) < 1e-2
    assert rel(x4.grad, x4r.grad) < 3e-2


@pytest.mark.parametrize("V,start,full", [(50304, 0, 50304), (1000, 1000, 3000), (257, 0, 257)])
def test_cross_entropy(V, start, full):
    from gpt_neox_b200.ops.cross_entropy import _combine_stats, vocab_parallel_cross_entropy
    torch.manual_seed(7)
    rows = 300
    logits = bf(rows, V, scale=2.0, grad=True)
    labels = torch.randint(0, full, (rows,), device=DEV)
    if full == V:
        loss = vocab_parallel_cross_entropy(logits, labels, start)
        lr = logits.detach().float().requires_grad_(True)
        ref = F.cross_entropy(lr, labels, reduction="none")
        assert rel(loss, ref) < 1e-3
        w = torch.rand(rows, device=DEV)
        (loss * w).sum().backward()
        (ref * w).sum().backward()
        assert rel(logits.grad, lr.grad) < 2e-2
    else:
        # a shard of a larger vocabulary: (max, sumexp, target) statistics must match
        from gpt_neox_b200.ops import _lib
        stats = torch.empty(rows, 3, device=DEV)
        _lib.check(_lib.lib(logits).nx_ce_fwd(_lib.ptr(logits), _lib.ptr(labels), _lib.ptr(stats), rows, V, V, start, 0,
                                        _lib.stream()))
        lf = logits.detach().float()
        m = lf.max(-1).values
        s = torch.exp(lf - m[:, None]).sum(-1)
        loc = labels - start
        inside = (loc >= 0) & (loc < V)
        t = torch.where(inside, lf.gather(-1, loc.clamp(0, V - 1)[:, None]).squeeze(-1), torch.zeros_like(m))
        assert rel(stats[:, 0], m) < 1e-5 and rel(stats[:, 1], s) < 1e-3 and rel(stats[:, 2], t) < 1e-5


def test_adamw_sumsq_clip():
    from gpt_neox_b200.ops.optim import adamw_step_, clip_coef_, sumsq_
    torch.manual_seed(8)
    n = 100003
    p = torch.randn(n, device=DEV)
    pr = p.clone().requires_grad_(True)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    lp = torch.empty(n, device=DEV, dtype=DT)
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(DT)
        acc = torch.zeros(2, device=DEV)
        sumsq_(g, acc)
        assert rel(acc[0], g.float().pow(2).sum()) < 1e-3
        out, skip = torch.ones(2, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
        clip_coef_(acc, 1.0, 0.5, out, skip)
        norm = g.float().norm() * 0.5
        coef = min(1.0, 1.0 / (norm.item() + 1e-6)) * 0.5
        assert abs(out[0].item() - coef) / coef < 1e-3 and skip.item() == 0
        adamw_step_(p, m, v, g, lp, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                    grad_scale=out, skip=skip)
        pr.grad = g.float() * coef
        opt.step()
        assert rel(p, pr.detach()) < 1e-4
        assert rel(lp, pr.detach()) < 1e-2
    # non-finite gradients set the skip flag and the update is a no-op
    g = torch.full((n,), float("inf"), device=DEV).to(DT)
    acc = torch.zeros(2, device=DEV)
    sumsq_(g, acc)
    clip_coef_(acc, 1.0, 1.0, out, skip)
    assert skip.item() == 1
    before = p.clone()
    adamw_step_(p, m, v, g, lp, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=4,
                grad_scale=out, skip=skip)
    assert torch.equal(before, p)


def test_adamw_8bit_state_kernel_matches_the_pytorch_statement():
    """csrc/optim.cu adam8_kernel against ops/optim.py's PyTorch statement of the same update and the same 8-bit
    block-wise codes: the master weights agree to fp32 rounding, the codes agree except where a value sits on a
    rounding boundary of the logarithmic code (one step apart)."""
    from gpt_neox_b200.ops.optim import adamw8bit_step_, q8_blocks
    torch.manual_seed(9)
    n = 2048 * 5 + 1024
    p = torch.randn(n, device=DEV)
    pc = p.cpu().clone()
    st = [torch.zeros(n, dtype=torch.uint8), torch.zeros(n, dtype=torch.uint8), torch.zeros(q8_blocks(n)),
          torch.zeros(q8_blocks(n))]
    sg = [t.to(DEV) for t in st]
    lp = torch.empty(n, device=DEV, dtype=DT)
    scale = torch.tensor([0.5], device=DEV)
    skip = torch.zeros(1, dtype=torch.int32, device=DEV)
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    for step in range(1, 5):
        g = (torch.randn(n, device=DEV) * torch.rand(n, device=DEV) ** 3).to(DT)
        adamw8bit_step_(p, *sg, g, lp, step=step, grad_scale=scale, skip=skip, **kw)
        adamw8bit_step_(pc, *st, g.cpu(), None, step=step, grad_scale=torch.tensor([0.5]), **kw)
        assert rel(p.cpu(), pc) < 1e-5
        assert rel(lp.cpu(), pc) < 1e-2
        for a, b in ((sg[0], st[0]), (sg[1], st[1])):
            d = (a.cpu().to(torch.int32) & 127) - (b.to(torch.int32) & 127) if a is sg[0] else \
                a.cpu().to(torch.int32) - b.to(torch.int32)
            assert d.abs().max().item() <= 1 and (d != 0).float().mean().item() < 0.02
            b.copy_(a.cpu())                     # continue from identical codes so that the steps stay comparable
        assert rel(sg[2].cpu(), st[2]) < 1e-5 and rel(sg[3].cpu(), st[3]) < 1e-5
    skip.fill_(1)
    before = p.clone()
    adamw8bit_step_(p, *sg, g, lp, step=5, grad_scale=scale, skip=skip, **kw)
    assert torch.equal(before, p)


@pytest.mark.parametrize("hn,rot", [(128, 32), (96, 24), (64, 64)])
def test_rope_strided(hn, rot):
    from gpt_neox_b200.ops.rope import apply_rotary, rotary_tables
    torch.manual_seed(9)
    s, b, h = 50, 3, 4
    qkv = bf(s, b, h, 3 * hn)
    q = qkv[..., :hn].detach().requires_grad_(True)     # strided view
    cos, sin = rotary_tables(rot, 64, device=DEV)
    y = apply_rotary(q, cos, sin, rot, 5)
    g = bf(s, b, h, hn)
    y.backward(g)
    qr = qkv[..., :hn].detach().float().cpu().requires_grad_(True)
    yr = apply_rotary(qr, cos.cpu(), sin.cpu(), rot, 5)
    yr.backward(g.float().cpu())
    assert rel(y.cpu(), yr) < 1e-2
    assert rel(q.grad.cpu(), qr.grad) < 1e-2


def test_embedding_fwd_bwd():
    from gpt_neox_b200.ops.embedding import embedding
    torch.manual_seed(10)
    V, H = 500, 256
    table = bf(V, H, grad=True)
    ids = torch.randint(0, 1000, (4, 33), device=DEV)
    out = embedding(ids, table, vocab_start=250)
    loc = ids - 250
    inside = (loc >= 0) & (loc < V)
    tr = table.detach().float().requires_grad_(True)
    ref = F.embedding(loc.clamp(0, V - 1), tr) * inside[..., None]
    assert rel(out, ref) < 1e-3
    g = bf(4, 33, H)
    out.backward(g)
    ref.backward(g.float())
    assert rel(table.grad, tr.grad) < 2e-2


def test_mlp_gelu_fused():
    from gpt_neox_b200.ops.fused import mlp_gelu
    torch.manual_seed(11)
    x = bf(3, 70, 256, grad=True)
    w1, b1 = bf(1024, 256, scale=0.05, grad=True), bf(1024, scale=0.1, grad=True)
    w2, b2 = bf(256, 1024, scale=0.05, grad=True), bf(256, scale=0.1, grad=True)
    res = bf(3, 70, 256, grad=True)
    for kind in ("erf", "tanh"):
        for t in (x, w1, b1, w2, b2, res):
            t.grad = None
        y = mlp_gelu(x, w1, b1, w2, b2, residual=res, kind=kind)
        g = bf(3, 70, 256)
        y.backward(g)
        r = [t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2, res)]
        yr = F.linear(F.gelu(F.linear(r[0], r[1], r[2]), approximate="tanh" if kind == "tanh" else "none"),
                      r[3], r[4]) + r[5]
        yr.backward(g.float())
        assert rel(y, yr) < 2e-2
        for t, tr in zip((x, w1, b1, w2, b2, res), r):
            assert rel(t.grad, tr.grad) < 3e-2, kind


@pytest.mark.parametrize("np_,kvp,hn,rot", [(4, 4, 128, 32), (8, 2, 64, 64), (4, 4, 96, 24)])
def test_qkv_attention_fused(np_, kvp, hn, rot):
    from gpt_neox_b200.ops.fused import qkv_attention
    from gpt_neox_b200.ops.rope import rotary_tables
    torch.manual_seed(12)
    s, b = 300, 2
    width = (np_ + 2 * kvp) * hn
    qkv = bf(s, b, width, grad=True)
    cos, sin = rotary_tables(rot, 512, device=DEV)
    out = qkv_attention(qkv.clone(), num_heads=np_, num_kv_heads=kvp, head_dim=hn, rotary_dim=rot, cos=cos, sin=sin)
    qr = qkv.detach().float().cpu().requires_grad_(True)
    ref = qkv_attention(qr, num_heads=np_, num_kv_heads=kvp, head_dim=hn, rotary_dim=rot, cos=cos.cpu(),
                        sin=sin.cpu())
    assert rel(out.cpu(), ref) < 2e-2
    g = bf(s, b, np_ * hn)
    x = qkv.clone()
    o2 = qkv_attention(x, num_heads=np_, num_kv_heads=kvp, head_dim=hn, rotary_dim=rot, cos=cos, sin=sin)
    (gq,) = torch.autograd.grad(o2, x, g)
    ref.backward(g.float().cpu())
    assert rel(gq.cpu(), qr.grad) < 3e-2


@pytest.mark.parametrize("cfg", [
    dict(b=2, sq=512, sk=512, h=4, hk=4, d=128), dict(b=1, sq=300, sk=300, h=4, hk=2, d=96),
    dict(b=1, sq=384, sk=384, h=2, hk=2, d=64), dict(b=1, sq=512, sk=512, h=2, hk=2, d=128, causal=False),
    dict(b=1, sq=512, sk=512, h=2, hk=2, d=128, window=100), dict(b=1, sq=512, sk=512, h=4, hk=4, d=128, alibi=True),
    dict(b=2, sq=64, sk=320, h=2, hk=1, d=64),
    # cached decoding: one new token (and a short chunk) against a long key sequence
    dict(b=2, sq=1, sk=700, h=4, hk=2, d=128), dict(b=1, sq=5, sk=261, h=2, hk=2, d=64, alibi=True),
    # dropout on the probabilities: the fp32 oracle applies the kernels' own mask
    dict(b=2, sq=512, sk=512, h=4, hk=4, d=128, dropout=0.1), dict(b=1, sq=300, sk=300, h=4, hk=2, d=64, dropout=0.25),
    dict(b=1, sq=384, sk=384, h=2, hk=2, d=128, dropout=0.5, alibi=True, window=200)])
def test_flash_attention(cfg):
    from gpt_neox_b200.ops.attention import alibi_slopes, attention_reference, flash_attention
    torch.manual_seed(13)
    b, sq, sk, h, hk, d = (cfg[k] for k in ("b", "sq", "sk", "h", "hk", "d"))
    causal, window = cfg.get("causal", True), cfg.get("window", -1)
    al = alibi_slopes(h).to(DEV) if cfg.get("alibi") else None
    q, k, v = bf(b, sq, h, d, grad=True), bf(b, sk, hk, d, grad=True), bf(b, sk, hk, d, grad=True)
    drop, seed = cfg.get("dropout", 0.0), 0x1234ABCD5678EF01
    o = flash_attention(q, k, v, causal=causal, window=window, alibi=al, dropout_p=drop, seed=seed)
    g = bf(b, sq, h, d)
    o.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    oref, _ = attention_reference(qr, kr, vr, causal=causal, window=window, alibi=al, dropout_p=drop, seed=seed)
    oref.backward(g.float())
    assert rel(o, oref) < 2e-2
    assert rel(q.grad, qr.grad) < 3e-2 and rel(k.grad, kr.grad) < 3e-2 and rel(v.grad, vr.grad) < 3e-2


@pytest.mark.parametrize("env", [{"NEOX_ATTN_FWD_SHAPE": "1"}, {"NEOX_ATTN_FWD_SHAPE": "3"},
                                 {"NEOX_ATTN_BWD_WARPS": "4"}, {"NEOX_ATTN_DKV_PIPE": "0", "NEOX_ATTN_DQ_PIPE": "0"}],
                         ids=["fwd_shape1", "fwd_shape3", "bwd_4warps", "bwd_unpipelined"])
def test_flash_attention_selectable_kernel_shapes(env):
    """The kernel shapes that an environment variable selects instead of the defaults (read once per process, hence a
    child process): the dense, dropout and block-sparse cases of this file under each of them."""
    import os
    import subprocess
    import sys
    if "_dtype" in globals() and DT != torch.bfloat16:
        pytest.skip("one operand type is enough for the shape selection")
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", os.path.abspath(__file__), "-k",
           "(test_flash_attention or test_block_sparse_flash_attention) and not selectable and not varlen"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=dict(os.environ, **env))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout


@pytest.mark.parametrize("kind,cfg,block,sq,sk", [
    ("sparse_fixed", {"num_local_blocks": 4, "num_global_blocks": 1}, 16, 640, 640),
    ("bigbird", {"num_sliding_window_blocks": 3, "num_global_blocks": 1, "num_random_blocks": 1}, 32, 512, 512),
    ("bslongformer", {"num_sliding_window_blocks": 3, "global_block_indices": [0]}, 64, 1024, 1024),
    ("local", {"num_local_blocks": 2}, 128, 1024, 1024),
    ("sparse_variable", {"local_window_blocks": [2, 4], "global_block_indices": [0]}, 16, 3, 500)])
def test_block_sparse_flash_attention(kind, cfg, block, sq, sk):
    """The five block-sparse layouts inside the flash kernels (key tiles without a live block are skipped, the rest
    masked per sub-block), forward and backward, against the fp32 oracle with the same token mask; the last case is
    cached decoding (3 new tokens against 500 keys)."""
    from gpt_neox_b200.models.sparse_attention import block_layout
    from gpt_neox_b200.ops.attention import BlockLayout, attention_reference, flash_attention
    torch.manual_seed(17)
    nb = (max(sq, sk) + block - 1) // block
    lay = BlockLayout(block_layout(kind, nb, dict(cfg, block=block), seed=3), block)
    rows, anyt = lay.tables(sq, sk, DEV)
    if sq >= 512:
        assert int((anyt == 0).sum()) > 0                     # some tiles really are skipped
    b, h, hk, d = 2, 4, 2, 64
    q, k, v = bf(b, sq, h, d, grad=True), bf(b, sk, hk, d, grad=True), bf(b, sk, hk, d, grad=True)
    o = flash_attention(q, k, v, causal=True, block_layout=lay)
    g = bf(b, sq, h, d)
    o.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    oref, _ = attention_reference(qr, kr, vr, causal=True, block_layout=lay)
    oref.backward(g.float())
    assert rel(o, oref) < 2e-2
    assert rel(q.grad, qr.grad) < 3e-2 and rel(k.grad, kr.grad) < 3e-2 and rel(v.grad, vr.grad) < 3e-2


def test_flash_attention_varlen_matches_per_sequence_oracle():
    """Packed sequences of unequal length (and unequal query / key lengths: cached decoding): each attends to itself only."""
    from gpt_neox_b200.ops.attention import attention_reference, flash_attention_varlen
    torch.manual_seed(31)
    lq, lk, h, hk, d = [130, 1, 257, 64], [130, 300, 257, 200], 4, 2, 64
    cq = [0] + torch.tensor(lq).cumsum(0).tolist()
    ck = [0] + torch.tensor(lk).cumsum(0).tolist()
    q, k, v = bf(cq[-1], h, d, grad=True), bf(ck[-1], hk, d, grad=True), bf(ck[-1], hk, d, grad=True)
    o = flash_attention_varlen(q, k, v, cq, torch.tensor(ck))
    g = bf(cq[-1], h, d)
    o.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    refs = [attention_reference(qr[cq[i]:cq[i + 1]][None], kr[ck[i]:ck[i + 1]][None], vr[ck[i]:ck[i + 1]][None])[0][0]
            for i in range(4)]
    oref = torch.cat(refs, 0)
    oref.backward(g.float())
    assert rel(o, oref) < 2e-2
    assert rel(q.grad, qr.grad) < 3e-2 and rel(k.grad, kr.grad) < 3e-2 and rel(v.grad, vr.grad) < 3e-2


def test_attention_dropout_mask_statistics_and_seed_dependence():
    """The mask is a pure function of (seed, batch, head, q, k): the keep rate matches 1 - p (p in steps of 1/256),
    rows and columns are not correlated, and another seed gives another mask."""
    from gpt_neox_b200.ops.attention import dropout_keep_mask, dropout_threshold
    for p in (0.1, 0.5):
        m = dropout_keep_mask(2, 3, 256, 384, p, 77, DEV).float()
        want = 1.0 - dropout_threshold(p) / 256.0
        assert abs(m.mean().item() - want) < 4e-3
        assert (m.mean(dim=-1) - want).abs().max().item() < 0.15 and (m.mean(dim=-2) - want).abs().max().item() < 0.17
        assert (m[0, 0] != m[0, 1]).float().mean().item() > 0.1            # heads differ
        m2 = dropout_keep_mask(2, 3, 256, 384, p, 78, DEV).float()
        assert (m != m2).float().mean().item() > 0.1                       # seeds differ


def test_qkv_attention_dropout_matches_the_oracle_with_the_same_mask():
    from gpt_neox_b200.ops.fused import qkv_attention
    from gpt_neox_b200.ops.rope import rotary_tables
    torch.manual_seed(21)
    s, b, np_, hn, rot = 256, 2, 4, 64, 16
    qkv = bf(s, b, 3 * np_ * hn, grad=True)
    cos, sin = rotary_tables(rot, 512, device=DEV)
    kw = dict(num_heads=np_, num_kv_heads=np_, head_dim=hn, rotary_dim=rot, dropout_p=0.2, seed=99)
    x = qkv.clone()
    out = qkv_attention(x, cos=cos, sin=sin, **kw)
    qr = qkv.detach().float().cpu().requires_grad_(True)
    ref = qkv_attention(qr, cos=cos.cpu(), sin=sin.cpu(), **kw)
    assert rel(out.cpu(), ref) < 2e-2
    g = bf(s, b, np_ * hn)
    (gq,) = torch.autograd.grad(out, x, g)
    ref.backward(g.float().cpu())
    assert rel(gq.cpu(), qr.grad) < 3e-2


def test_device_error_word_roundtrip():
    """The host can pre-set and read back the device error word (the fault-injection hook used by
    the failure-detection tests; no GPU wait is ever made to run out for it)."""
    from gpt_neox_b200.ops import _lib
    assert _lib.read_device_error(clear=True) == 0
    _lib.check(_lib.lib().nx_poison_device_error(0x301))
    with pytest.raises(_lib.DeviceWaitTimeout):
        _lib.raise_on_device_error()
    assert _lib.read_device_error(clear=False) == 0


def test_bias_and_norm_gradients_accumulate_straight_into_main_grad():
    """With an fp32 ``main_grad`` on the parameters (what the engine installs) the norm and bias-gradient kernels add
    into it themselves: nothing reaches ``.grad``, and two backward passes leave twice the fp32 reference there."""
    from gpt_neox_b200.ops.gemm import linear
    from gpt_neox_b200.ops.norm import dual_layer_norm
    torch.manual_seed(21)
    rows, H, N = 640, 1024, 768
    x = bf(rows, H, grad=True)
    params = {"g1": (1 + 0.1 * torch.randn(H, device=DEV)).to(DT), "b1": bf(H, scale=0.1), "g2": (1 + 0.1 * torch.randn(H, device=DEV)).to(DT),
              "b2": bf(H, scale=0.1), "w": bf(N, H, scale=0.05), "b": bf(N, scale=0.1)}
    for p in params.values():
        p.requires_grad_(True)
        p.main_grad = torch.zeros(p.shape, device=DEV, dtype=torch.float32)
    g = bf(rows, N)
    g2 = bf(rows, H)
    for _ in range(2):
        y1, y2 = dual_layer_norm(x, params["g1"], params["b1"], params["g2"], params["b2"], 1e-5)
        out = linear(y1, params["w"], params["b"])
        torch.autograd.backward([out, y2], [g, g2])
    ref = {k: v.detach().float().requires_grad_(True) for k, v in params.items()}
    xr = x.detach().float().requires_grad_(True)
    r1 = F.layer_norm(xr, (H,), ref["g1"], ref["b1"], 1e-5)
    r2 = F.layer_norm(xr, (H,), ref["g2"], ref["b2"], 1e-5)
    ro = F.linear(r1.to(DT).float(), ref["w"], ref["b"])
    torch.autograd.backward([ro, r2], [g.float(), g2.float()])
    for k, p in params.items():
        assert p.grad is None, k
        assert rel(p.main_grad, 2 * ref[k].grad) < 2e-2, k
