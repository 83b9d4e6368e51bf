"""Timings of the fused tensor-parallel GEMM + collective kernels against their parts, on the launched ranks:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m gpt_neox_b200.comm.bench_fused [--model pythia-6-9B|neox-20B] [--iters 20] [--json out.json]

For the column-parallel (all-gather -> GEMM) and row-parallel (GEMM -> reduce-scatter, GEMM -> all-reduce)
linears of one transformer layer it reports, per op: the fused kernel, the same GEMM alone on already gathered
data (what the collective costs on top), and the unfused pair (this library's GEMM + the NCCL collective).
CUDA events on the launching stream, max over ranks; two operand sets are alternated so that every iteration
reads its operands from HBM, not from L2.  Roofline per op: max(FLOPs / bf16 peak, bytes over NVLink / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

SHAPES = {"pythia-6-9B": dict(tokens=8192, h=4096, ffn=16384), "neox-20B": dict(tokens=4096, h=6144, ffn=24576)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="pythia-6-9B", choices=sorted(SHAPES))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--peak-tflops", type=float, default=1623.7, help="burst bf16 GEMM peak of the device (TFLOP/s)")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="NVLink bandwidth per direction (GB/s)")
    args = ap.parse_args(argv)
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from . import symm
    from ..ops.gemm import gemm
    be = symm.init_group(dist.group.WORLD)
    sh = SHAPES[args.model]
    M, h, f = sh["tokens"], sh["h"], sh["ffn"] // ws
    dt = torch.bfloat16
    torch.manual_seed(1 + rank)
    mk = lambda *s: [torch.randn(*s, device=dev).to(dt) for _ in range(2)]          # noqa: E731
    x_shard, x_full = mk(M // ws, h), mk(M, h)
    w_up, w_qkv = mk(f, h), mk(3 * h // ws, h)
    a_mlp, w_down = mk(M, f), mk(h, f)
    a_att, w_out = mk(M, h // ws), mk(h, h // ws)
    out_rs = torch.empty(M // ws, h, device=dev, dtype=dt)
    gath = torch.empty(M, h, device=dev, dtype=dt)

    def timeit(fn):
        for i in range(3):
            fn(i & 1)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.iters):
            fn(i & 1)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def nccl_ag_gemm(w):
        def fn(i):
            dist.all_gather_into_tensor(gath, x_shard[i])
            return gemm(gath, w[i])
        return fn

    def nccl_gemm_rs(a, w):
        def fn(i):
            dist.reduce_scatter_tensor(out_rs, gemm(a[i], w[i]))
        return fn

    def nccl_gemm_ar(a, w):
        def fn(i):
            y = gemm(a[i], w[i])
            dist.all_reduce(y)
        return fn

    ops = [
        ("ag_gemm qkv", lambda i: be.ag_gemm(x_shard[i], w_qkv[i]), lambda i: gemm(x_full[i], w_qkv[i]),
         nccl_ag_gemm(w_qkv), 2.0 * M * h * (3 * h // ws), (ws - 1) * (M // ws) * h * 2),
        ("ag_gemm mlp-up", lambda i: be.ag_gemm(x_shard[i], w_up[i]), lambda i: gemm(x_full[i], w_up[i]),
         nccl_ag_gemm(w_up), 2.0 * M * h * f, (ws - 1) * (M // ws) * h * 2),
        ("gemm_rs attn-out", lambda i: be.gemm_rs(a_att[i], w_out[i]), lambda i: gemm(a_att[i], w_out[i]),
         nccl_gemm_rs(a_att, w_out), 2.0 * M * h * (h // ws), (ws - 1) * (M // ws) * h * 2),
        ("gemm_rs mlp-down", lambda i: be.gemm_rs(a_mlp[i], w_down[i]), lambda i: gemm(a_mlp[i], w_down[i]),
         nccl_gemm_rs(a_mlp, w_down), 2.0 * M * h * f, (ws - 1) * (M // ws) * h * 2),
    ]
    if be.can_fuse_ar(M, f, h):
        ops.append(("gemm_ar mlp-down", lambda i: be.gemm_ar(a_mlp[i], w_down[i]), lambda i: gemm(a_mlp[i], w_down[i]),
                    nccl_gemm_ar(a_mlp, w_down), 2.0 * M * h * f, 2 * (ws - 1) * (M // ws) * h * 2))
    rows = []
    for name, fused, alone, unfused, flops, link_bytes in ops:
        t_f, t_a, t_u = timeit(fused), timeit(alone), timeit(unfused)
        roof = max(flops / (args.peak_tflops * 1e12), link_bytes / (args.link_gbs * 1e9)) * 1e3
        rows.append({"op": name, "fused_ms": t_f, "gemm_alone_ms": t_a, "gemm_plus_nccl_ms": t_u,
                     "overhead_vs_gemm": t_f / t_a - 1.0, "tflops": flops / t_f / 1e9, "nvlink_mb": link_bytes / 1e6,
                     "roofline_ms": roof, "fraction_of_roofline": roof / t_f})
    from ..ops import _lib
    err = _lib.read_device_error()
    if rank == 0:
        print(f"{args.model} layer shapes, {ws} ranks, tokens {M}, h {h}, ffn/rank {f}; device error word {err}")
        print(f"{'op':18s} {'fused':>9s} {'GEMM alone':>11s} {'GEMM+NCCL':>10s} {'over GEMM':>10s} {'TFLOP/s':>8s} {'roofline':>9s}")
        for r in rows:
            print(f"{r['op']:18s} {r['fused_ms']:8.3f}  {r['gemm_alone_ms']:10.3f}  {r['gemm_plus_nccl_ms']:9.3f}  "
                  f"{100 * r['overhead_vs_gemm']:8.1f}%  {r['tflops']:7.0f}  {r['fraction_of_roofline']:8.2f}")
        if args.json:
            with open(args.json, "w") as fh:
                json.dump({"model": args.model, "ranks": ws, "rows": rows}, fh, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
