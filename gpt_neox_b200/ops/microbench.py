"""Kernel microbenchmarks: ``python -m gpt_neox_b200.ops.microbench <op> [--shape ...]``.

Times one operator with CUDA events on the launching stream (3 warm-up runs, a 256 MiB write between
timed runs to flush L2, median of ``--iters``) and prints one JSON line with the achieved rate and its
fraction of the measured peaks (``MEASURED_PEAKS.json`` beside the package when present, otherwise the
numbers passed by ``--peak-tflops`` / ``--peak-gbs``).  ``--once`` runs the operator a few times without
timing: the form to put under a profiler.  ``--graph`` captures the operator's launches into a CUDA graph
first and times replays of it, which takes the Python and launch overhead of a many-launch operator
out of a microsecond-scale measurement.

ops: gemm, gemm_fp8, gemm_mxfp8, mxfp8_quantize, gemm_wgrad, attn_fwd, attn_bwd, layernorm, dual_norm_bwd, scan_fwd, scan_bwd, conv1d, moe_fwd, moe_fwdbwd,
     wkv_fwd, wkv_fwdbwd, adamw, ce   (moe: tokens = batch*seq, hidden --n, ffn --k, experts --heads, top-2)
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks(args):
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    tf, gbs, src = args.peak_tflops, args.peak_gbs, "flags"
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        tf, gbs, src = d.get("bf16_tflops", tf), d.get("hbm_gbs", gbs), "measured"
    return tf, gbs, src


def _time(fn, iters, flush=True):
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def build(op, a):
    """-> (callable, flops, bytes) for one launch group of ``op``."""
    dev, bf = "cuda", torch.bfloat16
    rn = lambda *s: torch.randn(*s, device=dev, dtype=bf)
    if op in ("gemm", "gemm_wgrad"):
        from .gemm import gemm
        M, N, K = a.m, a.n, a.k
        if op == "gemm":
            x, w = rn(M, K), rn(N, K)
            fn = lambda: gemm(x, w)
        else:
            x, g = rn(K, M), rn(K, N)            # wgrad: x^T g, the reduction runs over rows
            fn = lambda: gemm(x, g, trans_a=True, trans_b=True)
        return fn, 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    if op == "gemm_fp8":
        from . import fp8
        M, N, K = a.m, a.n, a.k
        ma, mb = fp8.Fp8TensorMeta(dev), fp8.Fp8TensorMeta(dev)
        x8, _ = fp8.quantize(rn(M, K), ma)
        w8, _ = fp8.quantize(rn(N, K), mb)
        alpha = torch.ones(1, device=dev)
        fn = lambda: fp8.gemm_fp8(x8, w8, alpha)
        return fn, 2.0 * M * N * K, 1.0 * (M * K + N * K) + 2.0 * M * N
    if op in ("gemm_mxfp8", "mxfp8_quantize"):
        from . import fp8
        M, N, K = a.m, a.n, a.k
        if op == "mxfp8_quantize":
            x = rn(M, N)
            fn = lambda: fp8.mxfp8_quantize(x)
            return fn, 0.0, 3.0 * M * N + 4.0 * M * N / 32
        x8, sx = fp8.mxfp8_quantize(rn(M, K))
        w8, sw = fp8.mxfp8_quantize(rn(N, K))
        fn = lambda: fp8.gemm_mxfp8(x8, sx, w8, sw)
        return fn, 2.0 * M * N * K, 1.0 * (M * K + N * K) + 2.0 * M * N
    if op in ("attn_fwd", "attn_bwd"):
        from .attention import flash_attention
        b, s, h, d = a.batch, a.seq, a.heads, a.head_dim
        q, k, v = (rn(b, s, h, d).requires_grad_(True) for _ in range(3))
        causal_flops = 4.0 * b * h * s * s * d / 2
        if op == "attn_fwd":
            def fn():
                with torch.no_grad():
                    flash_attention(q, k, v)
            return fn, causal_flops, 2.0 * 4 * b * s * h * d
        o = flash_attention(q, k, v)
        g = torch.ones_like(o)
        fn = lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True)
        return fn, 2.5 * causal_flops, 2.0 * 8 * b * s * h * d
    if op == "layernorm":
        from .norm import layer_norm
        x, w, b_ = rn(a.m, a.n), rn(a.n), rn(a.n)
        fn = lambda: layer_norm(x, w, b_, 1e-5)
        return fn, 0.0, 2.0 * 2 * a.m * a.n
    if op == "dual_norm_bwd":
        # backward of the parallel-residual block's two LayerNorms + the residual-stream gradient:
        # reads x, dy1, dy2, g_res and writes dx (five [m, n] bf16 passes); the kernel pair is launched
        # directly on preallocated buffers
        from . import _lib
        L = _lib.lib()
        x, g0, g1, g2, dx = (rn(a.m, a.n) for _ in range(5))
        w1, w2 = rn(a.n), rn(a.n)
        mean, rstd = torch.zeros(a.m, device=dev), torch.ones(a.m, device=dev)
        blocks = L.nx_norm_bwd_blocks(a.m)
        ws = torch.empty(blocks * 4 * a.n, device=dev)
        dg = [torch.empty(a.n, device=dev) for _ in range(4)]
        P = _lib.ptr
        fn = lambda: _lib.check(L.nx_norm_bwd(0, P(g1), P(g2), P(x), P(mean), P(rstd), P(w1), P(w2), P(g0), P(dx),
                                              P(dg[0]), P(dg[1]), P(dg[2]), P(dg[3]), P(ws), a.m, a.n, 0,
                                              _lib.stream()), "nx_norm_bwd")
        return fn, 0.0, 2.0 * 5 * a.m * a.n
    if op in ("scan_fwd", "scan_bwd", "conv1d"):
        from .mamba import causal_conv1d_silu, selective_scan
        B, L, D = a.batch, a.seq, a.n
        x, dt, z = (rn(L, B, D).transpose(0, 1) * 0.5 for _ in range(3))
        if op == "conv1d":
            w, bias = rn(D, 4), rn(D)
            def fn():
                with torch.no_grad():
                    causal_conv1d_silu(x, w, bias)
            return fn, 0.0, 2.0 * 2 * B * L * D
        Bm, Cm = rn(L, B, 16).transpose(0, 1), rn(L, B, 16).transpose(0, 1)
        A = -(torch.rand(D, 16, device=dev) * 4 + 0.5)
        Dp, dtb = torch.randn(D, device=dev), torch.randn(D, device=dev) - 2
        if op == "scan_fwd":
            def fn():
                with torch.no_grad():
                    selective_scan(x, dt, A, Bm, Cm, Dp, z, dtb)
            return fn, 0.0, 2.0 * 4 * B * L * D
        leaves = [t.detach().requires_grad_(True) for t in (x, dt, z)]
        y = selective_scan(leaves[0], leaves[1], A, Bm, Cm, Dp, leaves[2], dtb)
        g = torch.ones_like(y)
        fn = lambda: torch.autograd.grad(y, leaves, g, retain_graph=True)
        return fn, 0.0, 2.0 * 7 * B * L * D
    if op in ("moe_fwd", "moe_fwdbwd"):
        from .moe import experts_gelu
        T, k, E, h, ffn = a.batch * a.seq, 2, a.heads if a.heads <= 64 else 8, a.n, a.k
        x = rn(T, h).requires_grad_(True)
        w1 = (rn(E * ffn, h) * 0.05).requires_grad_(True)
        w2 = (rn(E * ffn, h) * 0.05).requires_grad_(True)
        wts, idx = torch.softmax(torch.randn(T, E, device=dev), -1).topk(k, dim=-1)
        wts = wts.to(bf)
        flops = 2.0 * 2 * T * k * h * ffn
        if op == "moe_fwd":
            def fn():
                with torch.no_grad():
                    experts_gelu(x, wts, idx, w1, w2, E)
            return fn, flops, 2.0 * (2 * E * ffn * h + 4 * T * k * h)
        def fn2():
            out = experts_gelu(x, wts, idx, w1, w2, E)
            torch.autograd.grad(out, (x, w1, w2), torch.ones_like(out))
        return fn2, 3 * flops, 2.0 * (2 * E * ffn * h + 4 * T * k * h) * 3
    if op in ("wkv_fwd", "wkv_fwdbwd"):
        from .wkv import wkv6
        B, T, H, N = a.batch, a.seq, a.heads, 64
        C = H * N
        mk = lambda: (rn(T, B, C) * 0.5).transpose(0, 1)
        r, k_, v = mk().requires_grad_(True), mk().requires_grad_(True), mk().requires_grad_(True)
        w = (rn(T, B, C) * 0.5 - 1.5).transpose(0, 1).requires_grad_(True)
        u = (torch.randn(H, N, device=dev) * 0.3).to(bf).requires_grad_(True)
        if op == "wkv_fwd":
            def fn():
                with torch.no_grad():
                    wkv6(r, k_, v, w, u)
            return fn, 4.0 * B * T * C * N, 2.0 * 5 * B * T * C
        def fn2():
            y = wkv6(r, k_, v, w, u)
            torch.autograd.grad(y, (r, k_, v, w, u), torch.ones_like(y))
        return fn2, 16.0 * B * T * C * N, 2.0 * 14 * B * T * C
    if op == "adamw":
        from . import optim as O
        n = a.m * a.n
        p, m, v = (torch.zeros(n, device=dev) for _ in range(3))
        g, lp = torch.randn(n, device=dev).to(bf), torch.zeros(n, device=dev, dtype=bf)
        scale = torch.ones(2, device=dev)
        skip = torch.zeros(1, device=dev, dtype=torch.int32)
        fn = lambda: O.adamw_step_(p, m, v, g, lp, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                   step=3, adam_w_mode=True, grad_scale=scale, skip=skip)
        return fn, 0.0, n * (3 * 4 * 2 + 2 + 2.0)
    if op == "ce":
        from .cross_entropy import vocab_parallel_cross_entropy
        logits = rn(a.m, a.n)
        tgt = torch.randint(0, a.n, (a.m,), device=dev)
        def fn():
            with torch.no_grad():
                vocab_parallel_cross_entropy(logits, tgt)
        return fn, 0.0, 2.0 * a.m * a.n
    raise SystemExit(f"unknown op {op}")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--once", action="store_true", help="run 3 times untimed (profiler form)")
    ap.add_argument("--graph", action="store_true", help="time replays of a CUDA graph of the operator")
    ap.add_argument("--peak-tflops", type=float, default=1590.0)
    ap.add_argument("--peak-gbs", type=float, default=6650.0)
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    fn, flops, nbytes = build(a.op, a)
    if a.once:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        print(json.dumps({"op": a.op, "ran": 3}))
        return
    if a.graph:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        fn = graph.replay
    ms = _time(fn, a.iters)
    tf, gbs, src = _peaks(a)
    out = {"op": a.op, "ms": round(ms, 4), "args": {k: v for k, v in vars(a).items() if k not in ("op", "once")}}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out[f"frac_of_{src}_bf16_peak"] = round(flops / ms / 1e9 / tf, 3)
    out["gbs_algorithmic"] = round(nbytes / ms / 1e6, 1)
    out[f"frac_of_{src}_hbm_copy"] = round(nbytes / ms / 1e6 / gbs, 3)
    from . import _lib
    out["device_error_word"] = _lib.read_device_error()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
