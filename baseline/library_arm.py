"""Whole-step library baseline for ``bench.py --impl library``.

The same NeoX-shaped decoder and the same optimizer step as the benchmark's own arm, written in
plain PyTorch on vendor / library kernels only: ``F.linear`` (cuBLAS), ``flash_attn_func``
(flash-attn 2, falling back to ``F.scaled_dot_product_attention``), ``F.layer_norm``, ``F.gelu``,
``torch.optim.AdamW(fused=True)`` and NCCL collectives at the call sites the reference uses them
(megatron/mpu/layers.py:186-212 embedding reduce, :567-576 all-gather before a column-parallel
GEMM, :773-779 reduce-scatter after a row-parallel one, megatron/mpu/cross_entropy.py:27-112 three
all-reduces, ZeRO-1 reduce-scatter of a flat gradient buffer + all-gather of the updated
parameters).  None of this package's kernels, engine or communication layer is imported here.  It
is NOT the reference implementation (which cannot be installed offline) and is never reported as
such: its JSON line says ``"impl": "library"``.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

try:                                             # flash-attn 2.x wheels in the image
    from flash_attn import flash_attn_func as _flash
except Exception:                                # noqa: BLE001
    _flash = None

SHAPES = {
    "pythia-6-9B": dict(layers=32, hidden=4096, heads=32, ffn=16384, vocab=50432, rotary_pct=0.25),
    "pythia-1-4B": dict(layers=24, hidden=2048, heads=16, ffn=8192, vocab=50304, rotary_pct=0.25),
}


# ----------------------------------------------------------------------------- tensor-parallel regions
class _GatherSeq(torch.autograd.Function):
    """Sequence-parallel all-gather along dim 0; backward is the reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        ws = dist.get_world_size(group)
        out = torch.empty((x.shape[0] * ws,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        ws = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] // ws,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterSeq(torch.autograd.Function):
    """Sum over the tensor-parallel group, scattered along dim 0; backward is the all-gather."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        ws = dist.get_world_size(group)
        out = torch.empty((x.shape[0] // ws,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        ws = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] * ws,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _VocabParallelCE(torch.autograd.Function):
    """Cross-entropy over vocabulary shards: max, target-logit and sum-exp all-reduces."""

    @staticmethod
    def forward(ctx, logits, target, v0, group):
        lf = logits.float()
        mx = lf.max(dim=-1).values
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        lf = lf - mx.unsqueeze(-1)
        local = target - v0
        inside = (local >= 0) & (local < logits.shape[-1])
        idx = local.clamp(0, logits.shape[-1] - 1)
        tl = lf.gather(-1, idx.unsqueeze(-1)).squeeze(-1) * inside
        dist.all_reduce(tl, group=group)
        ex = lf.exp_()
        se = ex.sum(-1)
        dist.all_reduce(se, group=group)
        ctx.save_for_backward(ex.div_(se.unsqueeze(-1)).to(logits.dtype), idx, inside)
        return se.log() - tl

    @staticmethod
    def backward(ctx, g):
        p, idx, inside = ctx.saved_tensors
        grad = p.float()
        grad.scatter_add_(-1, idx.unsqueeze(-1), -inside.float().unsqueeze(-1))
        return (grad * g.unsqueeze(-1)).to(p.dtype), None, None, None


def _rope(x, cos, sin, rot):
    """NeoX-style rotary embedding on the first ``rot`` dims of every head.  x: [s, b, np, hn]."""
    xr, xp = x[..., :rot], x[..., rot:]
    x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
    xr = xr * cos + torch.cat((-x2, x1), dim=-1) * sin
    return torch.cat((xr, xp), dim=-1)


class Layer(torch.nn.Module):
    def __init__(self, c, tp, dev):
        super().__init__()
        h, f, dt = c["hidden"], c["ffn"], torch.bfloat16
        self.h, self.np, self.hn = h, c["heads"] // tp, h // c["heads"]
        mk = lambda *s: torch.nn.Parameter(torch.randn(*s, device=dev, dtype=dt) * 0.02)   # noqa: E731
        z = lambda *s: torch.nn.Parameter(torch.zeros(*s, device=dev, dtype=dt))           # noqa: E731
        self.ln1_w, self.ln1_b = torch.nn.Parameter(torch.ones(h, device=dev, dtype=dt)), z(h)
        self.ln2_w, self.ln2_b = torch.nn.Parameter(torch.ones(h, device=dev, dtype=dt)), z(h)
        self.qkv_w, self.qkv_b = mk(3 * h // tp, h), z(3 * h // tp)
        self.out_w, self.out_b = mk(h, h // tp), z(h)
        self.up_w, self.up_b = mk(f // tp, h), z(f // tp)
        self.down_w, self.down_b = mk(h, f // tp), z(h)
        for p in (self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b, self.out_b, self.down_b):
            p.replicated = True

    def forward(self, x, cos, sin, rot, group):
        # x: [s / tp, b, h] (sequence-parallel shard when tp > 1)
        a = F.layer_norm(x, (self.h,), self.ln1_w, self.ln1_b)
        m = F.layer_norm(x, (self.h,), self.ln2_w, self.ln2_b)
        if group is not None:
            a, m = _GatherSeq.apply(a, group), _GatherSeq.apply(m, group)
        s, b = a.shape[0], a.shape[1]
        qkv = F.linear(a, self.qkv_w, self.qkv_b).view(s, b, self.np, 3 * self.hn)
        q, k, v = qkv.split(self.hn, dim=-1)
        q, k = _rope(q, cos, sin, rot), _rope(k, cos, sin, rot)
        if _flash is not None and q.is_cuda:
            o = _flash(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), causal=True)     # [b, s, np, hn]
            o = o.transpose(0, 1).reshape(s, b, self.np * self.hn)
        else:
            o = F.scaled_dot_product_attention(q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3),
                                               is_causal=True)
            o = o.permute(2, 0, 1, 3).reshape(s, b, self.np * self.hn)
        attn = F.linear(o, self.out_w)
        u = F.gelu(F.linear(m, self.up_w, self.up_b))
        mlp = F.linear(u, self.down_w)
        y = attn + mlp                                    # GPT-J residual: one reduction for both branches
        if group is not None:
            y = _ReduceScatterSeq.apply(y, group)
        return x + y + self.out_b + self.down_b


class Model(torch.nn.Module):
    def __init__(self, c, tp, tp_rank, group, dev, seq):
        super().__init__()
        self.c, self.tp, self.group = c, tp, group
        self.v_local = c["vocab"] // tp
        self.v0 = tp_rank * self.v_local
        dt = torch.bfloat16
        self.emb = torch.nn.Parameter(torch.randn(self.v_local, c["hidden"], device=dev, dtype=dt) * 0.02)
        self.layers = torch.nn.ModuleList([Layer(c, tp, dev) for _ in range(c["layers"])])
        self.lnf_w = torch.nn.Parameter(torch.ones(c["hidden"], device=dev, dtype=dt))
        self.lnf_b = torch.nn.Parameter(torch.zeros(c["hidden"], device=dev, dtype=dt))
        self.lnf_w.replicated = self.lnf_b.replicated = True
        self.head = torch.nn.Parameter(torch.randn(self.v_local, c["hidden"], device=dev, dtype=dt) * 0.02)
        hn = c["hidden"] // c["heads"]
        self.rot = int(hn * c["rotary_pct"])
        inv = 1.0 / (10000 ** (torch.arange(0, self.rot, 2, device=dev).float() / self.rot))
        fr = torch.outer(torch.arange(seq, device=dev).float(), inv)
        e = torch.cat((fr, fr), dim=-1)
        self.cos = e.cos().to(dt)[:, None, None, :]
        self.sin = e.sin().to(dt)[:, None, None, :]

    def forward(self, tokens, labels):
        # tokens, labels: [b, s]
        if self.tp > 1:
            local = tokens - self.v0
            ok = (local >= 0) & (local < self.v_local)
            x = F.embedding(local.clamp(0, self.v_local - 1), self.emb) * ok.unsqueeze(-1)
            x = _ReduceScatterSeq.apply(x.transpose(0, 1).contiguous(), self.group)      # [s / tp, b, h]
        else:
            x = F.embedding(tokens, self.emb).transpose(0, 1).contiguous()
        for layer in self.layers:
            x = layer(x, self.cos, self.sin, self.rot, self.group if self.tp > 1 else None)
        x = F.layer_norm(x, (self.c["hidden"],), self.lnf_w, self.lnf_b)
        if self.tp > 1:
            x = _GatherSeq.apply(x, self.group)
        logits = F.linear(x, self.head).transpose(0, 1)                                    # [b, s, v / tp]
        if self.tp > 1:
            loss = _VocabParallelCE.apply(logits, labels, self.v0, self.group)
        else:
            loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1), reduction="none")
        return loss.mean()


class Zero1AdamW:
    """Flat bf16 parameter / gradient buffers, ZeRO-1 over the data-parallel group, fp32 master weights and
    moments on each rank's shard, ``torch.optim.AdamW(fused=True)``, global-norm clipping."""

    def __init__(self, model, dp_group, dp, dp_rank, tp_group, tp, lr=1.2e-4, clip=1.0):
        self.dp_group, self.dp, self.tp_group, self.tp, self.clip = dp_group, dp, tp_group, tp, clip
        ps = [p for p in model.parameters()]
        dev = ps[0].device
        n = sum(p.numel() for p in ps)
        unit = dp * 128
        self.total = (n + unit - 1) // unit * unit
        self.flat = torch.zeros(self.total, dtype=torch.bfloat16, device=dev)
        self.grad = torch.zeros(self.total, dtype=torch.bfloat16, device=dev)
        self.rep_mask_ranges = []
        off = 0
        for p in ps:
            k = p.numel()
            self.flat[off:off + k].copy_(p.data.reshape(-1))
            p.data = self.flat[off:off + k].view(p.shape)
            p.grad = self.grad[off:off + k].view(p.shape)
            if getattr(p, "replicated", False):
                self.rep_mask_ranges.append((off, off + k))
            off += k
        self.replicated = [p for p in ps if getattr(p, "replicated", False)]
        self.shard = self.total // dp
        self.s0 = dp_rank * self.shard
        # fp32 master weights / moments of this rank's shard, in pieces of CHUNK elements so that the fp32 copy
        # of the gradient is only ever one piece long (the 6.9B model at tp1 would not fit otherwise)
        self.chunks = []
        for a in range(0, self.shard, self.CHUNK):
            b = min(self.shard, a + self.CHUNK)
            m = torch.nn.Parameter(self.flat[self.s0 + a:self.s0 + b].float())
            o = torch.optim.AdamW([m], lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
            self.chunks.append((a, b, m, o))
        self.tp_rank = dist.get_rank(tp_group) if tp > 1 else 0

    CHUNK = 1 << 28

    def step(self):
        if self.tp > 1 and self.replicated:          # sequence-parallel LayerNorm / bias gradients: sum over TP
            buf = torch.cat([p.grad.reshape(-1) for p in self.replicated])
            dist.all_reduce(buf, group=self.tp_group)
            o = 0
            for p in self.replicated:
                p.grad.copy_(buf[o:o + p.numel()].view_as(p.grad))
                o += p.numel()
        gs = self.grad[self.s0:self.s0 + self.shard]
        if self.dp > 1:
            dist.reduce_scatter_tensor(gs, self.grad, group=self.dp_group)
        tot = torch.zeros((), dtype=torch.float32, device=gs.device)
        for a, b, _m, _o in self.chunks:
            tot += gs[a:b].float().pow_(2).sum()
        if self.tp > 1 and self.tp_rank != 0:        # replicated parameters are counted by TP rank 0 only
            for a, b in self.rep_mask_ranges:
                lo, hi = max(a, self.s0) - self.s0, min(b, self.s0 + self.shard) - self.s0
                if hi > lo:
                    tot -= gs[lo:hi].float().pow_(2).sum()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(tot)
        norm = tot.sqrt() / self.dp                  # the reduce-scatter summed; the step uses the mean
        coef = torch.clamp(self.clip / (norm + 1e-6), max=1.0) / self.dp
        for a, b, m, o in self.chunks:
            m.grad = gs[a:b].float().mul_(coef)
            o.step()
            m.grad = None
            self.flat[self.s0 + a:self.s0 + b].copy_(m.data)
        if self.dp > 1:
            dist.all_gather_into_tensor(self.flat, self.flat[self.s0:self.s0 + self.shard].clone(), group=self.dp_group)
        self.grad.zero_()


def build(model_name, n_gpus, rank, dev, seq):
    """Returns (model, optimizer, tp, dp, dp_rank)."""
    c = SHAPES[model_name]
    tp = 1 if (n_gpus == 1 or "1-4B" in model_name) else 2      # Pythia-1.4B: pure data parallel, as in bench.py
    dp = n_gpus // tp
    tp_group = dp_group = None
    tp_rank, dp_rank = 0, 0
    if n_gpus > 1:
        for i in range(dp):                       # consecutive ranks form a tensor-parallel group
            g = dist.new_group(list(range(i * tp, (i + 1) * tp)))
            if rank // tp == i:
                tp_group = g
        for j in range(tp):
            g = dist.new_group(list(range(j, n_gpus, tp)))
            if rank % tp == j:
                dp_group = g
        tp_rank, dp_rank = rank % tp, rank // tp
    torch.manual_seed(1234 + tp_rank)
    model = Model(c, tp, tp_rank, tp_group, dev, seq)
    opt = Zero1AdamW(model, dp_group, dp, dp_rank, tp_group, tp)
    return model, opt, tp, dp, dp_rank


def flops_per_step(model_name, global_batch, seq):
    """The reference's FLOPs model without activation recomputation (megatron/logging.py:147-160)."""
    c = SHAPES[model_name]
    L, h, V = c["layers"], c["hidden"], c["vocab"]
    return 24 * 3 * global_batch * seq * L * h * h * (1.0 + seq / (6.0 * h) + V / (16.0 * L * h))


def train_step(model, opt, batches):
    """One optimizer step over ``len(batches)`` micro-batches of [b, s + 1] token tensors on the device."""
    gas = len(batches)
    total = None
    for t in batches:
        loss = model(t[:, :-1], t[:, 1:]) / gas
        loss.backward()
        total = loss.detach() if total is None else total + loss.detach()
    opt.step()
    return total


__all__ = ["SHAPES", "build", "train_step", "flops_per_step", "math"]
