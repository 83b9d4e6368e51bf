"""Op-level checks of the NVLink communication layer on the visible GPUs (launched by torchrun, one rank per GPU).

Every fused GEMM + collective (all-gather -> GEMM, GEMM -> reduce-scatter, GEMM -> all-reduce), the stand-alone
peer-memory collectives, the ZeRO workspace and the expert-parallel dispatch / combine are compared with a plain
fp32 PyTorch product / reduction whose operands travel over NCCL.  Rank 0 prints ``CHECKS {json}``; any mismatch
raises on the rank that sees it (the job then exits non-zero).
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def close(out, ref, what, max_tol=2e-2, mean_tol=8e-3):
    """The tolerances of the single-GPU GEMM tests: maximum error relative to the largest value, mean relative error."""
    out, ref = out.float(), ref.float()
    err = (out - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
    mean = ((out - ref).abs().mean() / (ref.abs().mean() + 1e-6)).item()
    assert err < max_tol and mean < mean_tol, f"{what}: max err {err:.4g}, mean rel err {mean:.4g}"
    return err


def nccl_gather_rows(x, group):
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def main():
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}[sys.argv[1] if len(sys.argv) > 1 else "bf16"]
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    from gpt_neox_b200.comm import symm
    from gpt_neox_b200.ops import _lib
    be = symm.init_group(group)
    done = {}
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device=dev, generator=g) * scale).to(dtype)   # noqa: E731

    # ---- all-gather -> GEMM: several 256-row tiles per rank chunk, N not a multiple of the 256-wide tile, and a
    #      row count whose chunks are 128-row tiles only (the single-CTA kernel)
    for tag, m_shard, k, n, tb in (("pair", 512, 1088, 1000, False), ("pair_nn", 256, 512, 776, True),
                                   ("single", 384, 320, 520, False)):
        x = rnd(m_shard, k)
        w = rnd(k, n, scale=0.05) if tb else rnd(n, k, scale=0.05)
        dist.broadcast(w, 0)
        bias = rnd(n)
        dist.broadcast(bias, 0)
        assert be.can_fuse(m_shard * ws, k, n)
        y, gathered = be.ag_gemm(x, w, trans_b=tb, bias=bias)
        xf = nccl_gather_rows(x, group)
        ref = xf.float() @ (w.float() if tb else w.float().t()) + bias.float()
        assert torch.equal(gathered, xf), f"ag_gemm[{tag}]: gathered operand differs from the NCCL all-gather"
        done[f"ag_gemm_{tag}"] = close(y, ref, f"ag_gemm[{tag}]")

    # ---- GEMM -> reduce-scatter (+ residual in the epilogue, + bias and a second residual on the owner)
    for tag, m, k, n, tb in (("pair", 512 * ws, 576, 1000, False), ("pair_nn", 256 * ws, 1024, 520, True),
                             ("single", 384 * ws, 320, 264, False)):
        a = rnd(m, k)
        w = rnd(k, n, scale=0.05) if tb else rnd(n, k, scale=0.05)
        bias = rnd(n)
        dist.broadcast(bias, 0)
        res2 = rnd(m // ws, n)
        out = be.gemm_rs(a, w, trans_b=tb, bias=bias, residual2=res2)
        full = a.float() @ (w.float() if tb else w.float().t())
        dist.all_reduce(full, group=group)
        rows = m // ws
        ref = full[rank * rows:(rank + 1) * rows] + bias.float() + res2.float()
        done[f"gemm_rs_{tag}"] = close(out, ref, f"gemm_rs[{tag}]")

    # ---- GEMM -> all-reduce (tensor parallelism without sequence parallelism)
    m, k, n = 256 * ws * 2, 448, 1000
    if be.can_fuse_ar(m, k, n):
        a, w = rnd(m, k), rnd(n, k, scale=0.05)
        bias = rnd(n)
        dist.broadcast(bias, 0)
        out = be.gemm_ar(a, w, bias=bias).clone()
        full = a.float() @ w.float().t()
        dist.all_reduce(full, group=group)
        done["gemm_ar"] = close(out, full + bias.float(), "gemm_ar")

    # ---- the autograd functions of the fused linears: without grad (no pool slot is asked for), with an input that
    #      needs no gradient (none either), and the training case (gathered operand kept in a pool slot)
    from gpt_neox_b200.ops import fused_tp
    m_shard, k, n = 256, 512, 384
    w0 = rnd(n, k, scale=0.05)
    dist.broadcast(w0, 0)
    b0 = rnd(n)
    dist.broadcast(b0, 0)
    x0 = rnd(m_shard, k)
    xf = nccl_gather_rows(x0, group).float()
    ref = xf @ w0.float().t() + b0.float()
    with torch.no_grad():
        done["ag_linear_no_grad"] = close(fused_tp.ag_linear(x0, w0, b0, be), ref, "ag_linear under no_grad")
    wp, bp = w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    y = fused_tp.ag_linear(x0, wp, bp, be)                                   # x needs no gradient
    gy = rnd(m_shard * ws, n)
    dist.broadcast(gy, 0)
    y.backward(gy)
    done["ag_linear_weight_only"] = close(wp.grad, gy.float().t() @ xf, "ag_linear dW (input without grad)")
    xp, wp, bp = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    be.pool_release(be.pool_alloc(m_shard * ws * k * 2))                     # (creates the pool on first use)
    slots_before = len(be.pool["slots"].free) if be.pool else -1
    y = fused_tp.ag_linear(xp, wp, bp, be)
    in_use = (slots_before - len(be.pool["slots"].free)) if be.pool else 0
    y.backward(gy)
    done["ag_linear_train"] = close(y, ref, "ag_linear forward")
    close(wp.grad, gy.float().t() @ xf, "ag_linear dW")
    dx_full = gy.float() @ w0.float()
    dist.all_reduce(dx_full, group=group)                                    # every rank holds the same dY: sum = ws x
    close(xp.grad, dx_full[rank * m_shard:(rank + 1) * m_shard], "ag_linear dX (reduce-scattered)")
    close(bp.grad, gy.float().sum(0), "ag_linear db", 2e-2, 1e-2)
    if be.pool:
        assert in_use == 1 and len(be.pool["slots"].free) == slots_before, "pool slot not taken / not given back"
    done["gather_pool_slots"] = float(be.pool["n"]) if be.pool else 0.0

    # ---- stand-alone collectives over peer memory (16-bit and fp32)
    for dt, tag in ((dtype, "h16"), (torch.float32, "f32")):
        x = (torch.randn(ws * 96, 1000, device=dev, generator=g)).to(dt)
        ref = x.clone().float()
        dist.all_reduce(ref, group=group)
        got = be.all_reduce(x.clone())
        done[f"all_reduce_{tag}"] = close(got, ref, f"all_reduce[{tag}]", 1e-2, 4e-3)
        rs = be.reduce_scatter0(x.clone())
        rows = x.shape[0] // ws
        done[f"reduce_scatter_{tag}"] = close(rs, ref[rank * rows:(rank + 1) * rows], f"reduce_scatter0[{tag}]", 1e-2, 4e-3)
        ag = be.all_gather0(x[:rows].contiguous())
        assert torch.equal(ag, nccl_gather_rows(x[:rows].contiguous(), group)), f"all_gather0[{tag}]"
        done[f"all_gather_{tag}"] = 0.0

    # ---- ZeRO workspace: in-place gradient reduce-scatter and parameter all-gather
    n_el = ws * 256 * 37
    for gdt, tag in ((torch.float32, "f32"), (dtype, "h16")):
        esz = torch.empty((), dtype=gdt).element_size()
        zw = symm.ZeroWorkspace(group, n_el * esz, n_el * 2)
        grads = zw.grad_buffer(gdt)
        grads.copy_(torch.randn(n_el, device=dev, generator=g).to(gdt))
        ref = grads.clone().float()
        dist.all_reduce(ref, group=group)
        dist.barrier(group)
        zw.reduce_scatter_grads(gdt)
        torch.cuda.synchronize()
        shard = n_el // ws
        done[f"zero_rs_{tag}"] = close(grads[rank * shard:(rank + 1) * shard], ref[rank * shard:(rank + 1) * shard],
                                       f"zero reduce-scatter[{tag}]", 1e-2, 4e-3)
        # bucket-wise reduction (overlap_comm): odd ranges that straddle chunk borders, on a side stream, in place
        fresh = torch.randn(n_el, device=dev, generator=g).to(gdt)
        dist.barrier(group)
        grads.copy_(fresh)
        ref = fresh.clone().float()
        dist.all_reduce(ref, group=group)
        torch.cuda.synchronize()
        dist.barrier(group)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        cuts = [0, 64 * 5, shard - 64, shard + 64 * 3, n_el - 64 * 7, n_el]
        with torch.cuda.stream(side):
            for lo, hi in zip(cuts[:-1], cuts[1:]):
                zw.reduce_grad_range(gdt, lo * esz, hi * esz)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        done[f"zero_range_{tag}"] = close(grads[rank * shard:(rank + 1) * shard], ref[rank * shard:(rank + 1) * shard],
                                          f"zero bucket reduction[{tag}]", 1e-2, 4e-3)
        params = zw.param_buffer(dtype)
        params.zero_()
        mine = torch.randn(shard, device=dev, generator=g).to(dtype)
        params[rank * shard:(rank + 1) * shard].copy_(mine)
        dist.barrier(group)
        zw.all_gather_params()
        torch.cuda.synchronize()
        dist.barrier(group)
        assert torch.equal(params, nccl_gather_rows(mine, group)), f"zero all-gather[{tag}]"
        done[f"zero_ag_{tag}"] = 0.0
        assert zw.check_guards(), "a ZeRO kernel wrote into a guard band"
        del zw

    # ---- vocabulary-parallel embedding whose rows are stored straight into their consumers' buffers
    V, H, B, S = 64 * ws + 24, 264, 3, 16 * ws
    gt = torch.Generator(device="cuda").manual_seed(11)                     # table and ids: the same on all ranks
    table = torch.randn(V, H, device=dev, generator=gt).to(dtype)
    ids = torch.randint(0, V, (B, S), device=dev, generator=gt)
    per = (V + ws - 1) // ws
    lo, hi = rank * per, min(V, (rank + 1) * per)
    local = table[lo:hi].contiguous()
    want = torch.nn.functional.embedding(ids, table)
    for _ in range(2):                                                       # twice: the buffer is reused
        assert be.can_embed_push(ids, local, False) and be.can_embed_push(ids, local, True)
        assert torch.equal(be.embed_push(ids, local, lo, False), want), "embed_push: full output"
        s_loc = S // ws
        assert torch.equal(be.embed_push(ids, local, lo, True), want[:, rank * s_loc:(rank + 1) * s_loc]), \
            "embed_push: sequence-parallel slice"
        ids = ids.flip(1).contiguous()
        want = torch.nn.functional.embedding(ids, table)
    done["embed_push"] = 0.0

    # ---- expert parallelism: dispatch / combine as peer loads against the fp32 statement of the experts
    from gpt_neox_b200.ops import moe_ep
    T, topk, H, ffn, E = 512, 2, 256, 512, 2 * ws
    e_local = E // ws
    x = rnd(T, H)
    logits = torch.randn(T, E, device=dev, generator=g)
    wts, idx = torch.softmax(logits, -1).topk(topk, dim=-1)
    wts = wts.to(dtype)
    gw = torch.Generator(device="cuda").manual_seed(5)                      # the full expert weights, same on all ranks
    w1_all = (torch.randn(E * ffn, H, device=dev, generator=gw) * 0.05).to(dtype)
    w2_all = (torch.randn(E * ffn, H, device=dev, generator=gw) * 0.05).to(dtype)
    w1 = w1_all[rank * e_local * ffn:(rank + 1) * e_local * ffn].contiguous()
    w2 = w2_all[rank * e_local * ffn:(rank + 1) * e_local * ffn].contiguous()
    out = moe_ep.experts_gelu_ep(x, wts, idx, w1, w2, E, group, "erf")
    ref = torch.zeros(T, H, device=dev)
    xf = x.float()
    for e in range(E):
        h = torch.nn.functional.gelu(xf @ w1_all[e * ffn:(e + 1) * ffn].float().t()).to(dtype).float()
        ye = (h @ w2_all[e * ffn:(e + 1) * ffn].float()).to(dtype).float()
        for j in range(topk):
            sel = idx[:, j] == e
            ref[sel] += wts[sel, j].float()[:, None] * ye[sel]
    done["moe_ep"] = close(out, ref, "expert-parallel dispatch / combine", 3e-2, 1.5e-2)

    torch.cuda.synchronize()
    assert be.check_guards(), "a kernel wrote into a guard band of the symmetric workspace"
    done["guards_intact"] = 0.0
    done["debug_bounds_build"] = float(_lib.lib().nx_comm_debug_bounds())
    err = _lib.read_device_error()
    assert err == 0, f"device error word 0x{err:x}"
    dist.barrier()
    if rank == 0:
        print("CHECKS " + json.dumps({"ws": ws, "dtype": str(dtype), "checks": done}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
