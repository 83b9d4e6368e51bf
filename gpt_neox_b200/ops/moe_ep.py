"""Expert-parallel dropless MoE over NVLink peer memory (csrc/moe_ep.cu): the dispatch all-to-all is folded
into the permutation gather and the combine all-to-all into the weighted un-permutation, both as plain peer
loads from the other ranks' symmetric workspaces.  No NCCL call and no host read of the routing result.

One layer call on every rank of the expert-parallel group::

    publish tokens + expert ids  | barrier |  plan (all ranks' copies -> local experts), pull-gather,
    grouped GEMMs, publish result rows + copy->row table  | barrier |  pull-combine

and the mirror image in backward.  The phases are separate functions so that a single-GPU test can drive the
workspaces of several emulated ranks in lockstep (kernels that wait on one another must not run as separate
launches on one GPU, so the emulation has no barrier kernel: stream order stands in for it).
Reference path: megatron/model/moe.py:85-160 + mpu/mappings.py:147-183.
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from . import _lib
from .gemm import LAUNCHES
from .moe import Plan, grouped_gemm_rows, grouped_wgrad

_DECLARED = False


def _declare():
    global _DECLARED
    L = _lib.lib()
    if not _DECLARED:
        P, I, LL, U = C.c_void_p, C.c_int, C.c_longlong, C.c_uint
        PP = C.POINTER(C.c_ulonglong)
        sigs = {"nx_moe_ep_flag_bytes": [], "nx_moe_ep_barrier": [PP, I, I, U, P],
                "nx_moe_ep_stage_ids": [PP, I, LL, I, I, I, P, P],
                "nx_moe_ep_gather": [PP, I, LL, LL, P, I, I, P, I, I, P, P, P],
                "nx_moe_ep_combine": [PP, I, I, LL, LL, LL, P, I, I, I, P, P, I, I, P, P]}
        for name, argtypes in sigs.items():
            for nm in (name, name + "_f16"):        # the bf16 build and the fp16 build
                f = getattr(L, nm)
                f.argtypes, f.restype = argtypes, I
        _DECLARED = True
    return L


def _layout(ws, T, k, H, e_local):
    """Byte offsets of the workspace regions (identical on every rank)."""
    L = _declare()
    al = lambda n: (n + 255) // 256 * 256
    Ck = T * k
    max_rows = L.nx_moe_max_rows(ws * Ck, e_local)
    off, o = {}, L.nx_moe_ep_flag_bytes()
    for name, nbytes in (("idx", 4 * Ck), ("wf", 2 * Ck), ("tok", 2 * T * H), ("dest", 4 * ws * Ck),
                         ("aux", 4 * max_rows), ("rows", 2 * max_rows * H)):
        off[name] = o
        o += al(nbytes)
    return off, o, max_rows


class EpWorkspace:
    """One rank's symmetric workspace and its view of the peers'."""

    def __init__(self, buf, ptrs, me, ws, T, k, H, e_local, barrier, dtype=torch.bfloat16):
        self.buf, self.me, self.ws, self.T, self.k, self.H, self.e_local = buf, me, ws, T, k, H, e_local
        self.Ck = T * k
        self.off, self.nbytes, self.max_rows = _layout(ws, T, k, H, e_local)
        self.ptrs = (C.c_ulonglong * 8)(*([int(p) for p in ptrs] + [0] * (8 - ws)))
        self.use_barrier = barrier
        self.dtype = dtype           # 16-bit dtype of tokens, routing weights and expert rows
        self.epoch = 0
        v = lambda name, n, dt: buf[self.off[name]:self.off[name] + n * torch.empty(0, dtype=dt).element_size()].view(dt)
        self.idx = v("idx", self.Ck, torch.int32)
        self.wf = v("wf", self.Ck, dtype)
        self.tok = v("tok", T * H, dtype).view(T, H)
        self.dest = v("dest", ws * self.Ck, torch.int32)
        self.aux = v("aux", self.max_rows, torch.float32)
        self.rows = v("rows", self.max_rows * H, dtype).view(self.max_rows, H)

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, group, T, k, H, e_local, dtype=torch.bfloat16):
        """Collective over ``group``: allocate and exchange the symmetric buffers."""
        import torch.distributed._symmetric_memory as symm_mem
        ws, me = dist.get_world_size(group), dist.get_rank(group)
        _, nbytes, _ = _layout(ws, T, k, H, e_local)
        dev = torch.device("cuda", torch.cuda.current_device())
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        buf[: _declare().nx_moe_ep_flag_bytes()].zero_()
        torch.cuda.synchronize()
        hdl = symm_mem.rendezvous(buf, group)
        w = cls(buf, hdl.buffer_ptrs, me, ws, T, k, H, e_local, barrier=True, dtype=dtype)
        w.hdl = hdl
        dist.barrier(group)
        return w

    @classmethod
    def emulated(cls, ws, T, k, H, e_local, device="cuda", dtype=torch.bfloat16):
        """``ws`` workspaces on ONE device, for driving emulated ranks in lockstep without barrier kernels."""
        _, nbytes, _ = _layout(ws, T, k, H, e_local)
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(ws)]
        ptrs = [b.data_ptr() for b in bufs]
        return [cls(bufs[r], ptrs, r, ws, T, k, H, e_local, barrier=False, dtype=dtype) for r in range(ws)]

    def fits(self, T, k, H, e_local, dtype=torch.bfloat16):
        return (T, k, H, e_local, dtype) == (self.T, self.k, self.H, self.e_local, self.dtype)

    # ------------------------------------------------------------------ kernels
    def barrier(self):
        if not self.use_barrier:
            return
        self.epoch += 1
        LAUNCHES["n"] += 1
        _lib.check(_declare().nx_moe_ep_barrier(self.ptrs, self.me, self.ws, self.epoch, _lib.stream()),
                   "nx_moe_ep_barrier")

    def plan(self):
        """Routing plan of this rank's experts over the copies every rank has published."""
        ids = torch.empty(self.ws * self.Ck, device=self.buf.device, dtype=torch.int64)
        LAUNCHES["n"] += 1
        _lib.check(_declare().nx_moe_ep_stage_ids(self.ptrs, self.ws, self.off["idx"], self.Ck, self.me * self.e_local,
                                                  self.e_local, _lib.ptr(ids), _lib.stream()), "nx_moe_ep_stage_ids")
        return Plan(ids.view(-1, self.k), self.e_local)

    def gather(self, plan, scaled=False, dot_with=None):
        """Pull the published token rows of all ranks into the padded expert-sorted layout."""
        out = torch.empty((plan.max_rows, self.H), device=self.buf.device, dtype=self.dtype)
        LAUNCHES["n"] += 1
        _declare()
        _lib.check(_lib.lib(self.dtype).nx_moe_ep_gather(
            self.ptrs, self.ws, self.off["tok"], self.off["wf"] if scaled else -1, _lib.ptr(plan.src_copy), self.Ck,
            self.k, _lib.ptr(out), plan.max_rows, self.H, _lib.ptr(dot_with),
            _lib.ptr(self.aux) if dot_with is not None else None, _lib.stream()), "nx_moe_ep_gather")
        return out

    def combine(self, expert_ids_i32, weights=None, want_aux=False):
        """Pull this rank's tokens' expert results from their owners and sum the k copies."""
        out = torch.empty((self.T, self.H), device=self.buf.device, dtype=self.dtype)
        aux = torch.empty(self.Ck, device=self.buf.device, dtype=self.dtype) if want_aux else None
        LAUNCHES["n"] += 1
        _declare()
        _lib.check(_lib.lib(self.dtype).nx_moe_ep_combine(
            self.ptrs, self.ws, self.me, self.off["rows"], self.off["dest"], self.off["aux"] if want_aux else -1,
            _lib.ptr(expert_ids_i32), self.e_local, self.Ck, self.k, _lib.ptr(weights), _lib.ptr(out), self.T, self.H,
            _lib.ptr(aux), _lib.stream()), "nx_moe_ep_combine")
        return out, aux


# ---------------------------------------------------------------------- phases of one layer call
def fwd_publish(W: EpWorkspace, x2, indices):
    W.tok.copy_(x2)
    W.idx.copy_(indices.reshape(-1))


def fwd_experts(W: EpWorkspace, w1, w2, kind):
    plan = W.plan()
    ffn = w1.shape[0] // W.e_local
    xp = W.gather(plan)
    pre = torch.empty((plan.max_rows, ffn), device=xp.device, dtype=xp.dtype)
    h = grouped_gemm_rows(xp, w1, plan, ffn, trans_b=False, gelu=kind, aux_out=pre, aux_deriv=True)   # pre = gelu'(.)
    y = grouped_gemm_rows(h, w2, plan, w2.shape[1], trans_b=True)
    W.rows.copy_(y)
    W.dest.copy_(plan.dest_row)
    return plan, xp, pre, h, y


def fwd_combine(W: EpWorkspace, ids_i32, wf):
    return W.combine(ids_i32, wf)[0]


def bwd_publish(W: EpWorkspace, g, wf):
    W.tok.copy_(g)
    W.wf.copy_(wf)


def bwd_experts(W: EpWorkspace, plan, xp, pre, h, y, w1, w2, kind, need=(True, True)):
    dy = W.gather(plan, scaled=True, dot_with=y)            # also leaves <g, y> per row in W.aux
    dpre = grouped_gemm_rows(dy, w2, plan, w2.shape[0] // plan.E, trans_b=False, dgelu_aux=pre, dgelu="mul")
    dw2 = grouped_wgrad(h, dy, plan, w2) if need[1] else None
    dxp = grouped_gemm_rows(dpre, w1, plan, w1.shape[1], trans_b=True)
    dw1 = grouped_wgrad(dpre, xp, plan, w1) if need[0] else None
    W.rows.copy_(dxp)
    W.dest.copy_(plan.dest_row)
    return dw1, dw2


def bwd_combine(W: EpWorkspace, ids_i32):
    return W.combine(ids_i32, None, want_aux=True)          # (dx, d routing weights per copy)


class _ExpertsGeluEPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, weights, indices, w1, w2, W, kind):
        ids = indices.reshape(-1).to(torch.int32)
        wf = weights.reshape(-1).contiguous()
        fwd_publish(W, x2, ids)
        W.barrier()
        plan, xp, pre, h, y = fwd_experts(W, w1, w2, kind)
        W.barrier()
        out = fwd_combine(W, ids, wf)
        ctx.save_for_backward(xp, pre, h, y, wf, w1, w2, ids)
        ctx.plan, ctx.kind, ctx.W, ctx.w_shape = plan, kind, W, weights.shape
        return out

    @staticmethod
    def backward(ctx, g):
        xp, pre, h, y, wf, w1, w2, ids = ctx.saved_tensors
        W = ctx.W
        bwd_publish(W, g.contiguous(), wf)
        W.barrier()
        dw1, dw2 = bwd_experts(W, ctx.plan, xp, pre, h, y, w1, w2, ctx.kind,
                               need=(ctx.needs_input_grad[3], ctx.needs_input_grad[4]))
        W.barrier()
        dx, d_w = bwd_combine(W, ids)
        return dx, d_w.view(ctx.w_shape), None, dw1, dw2, None, None


_WORKSPACES = {}


def enabled() -> bool:
    return os.environ.get("NEOX_MOE_P2P", "1") != "0"


def workspace_for(group, T, k, H, e_local, dtype=torch.bfloat16):
    """The expert-parallel group's workspace (one per group, shared by all layers; re-created when the
    token count or layer shape changes: a collective, every rank takes the same branch)."""
    key = id(group)
    W = _WORKSPACES.get(key)
    if W is None or not W.fits(T, k, H, e_local, dtype):
        W = EpWorkspace.create(group, T, k, H, e_local, dtype=dtype)
        _WORKSPACES[key] = W
    return W


def reset():
    _WORKSPACES.clear()


def experts_gelu_ep(x2, weights, indices, w1, w2, num_experts, group, kind="erf"):
    """Expert-parallel ``ops.moe.experts_gelu``: x2 [T, h] bf16 local tokens; weights / indices [T, k] (global
    expert ids); w1, w2 [E_local * ffn, h] this rank's experts."""
    ws = dist.get_world_size(group)
    T, k = indices.shape
    W = workspace_for(group, T, k, x2.shape[1], num_experts // ws, x2.dtype)
    return _ExpertsGeluEPFn.apply(x2, weights.to(x2.dtype), indices, w1, w2, W, kind)
