"""Symmetric-memory workspaces and the collectives / fused GEMM+collective kernels that run on them.

One workspace per process group: the same number of bytes allocated on every rank and mapped into
every peer (handle exchange and mapping are done by ``torch.distributed._symmetric_memory``; the
kernels that use the peer pointers are this library's own, csrc/comm.cu and csrc/gemm_tcgen05.cu).
Layout: 64 KiB of epoch flags, then payload.  Epochs are monotone counters advanced identically on
every rank, so flags are never reset.  When the platform offers an NVLS multicast mapping its
address is passed to the kernels, which then use ``multimem`` reductions / stores through the switch;
``NEOX_NVLS=0`` forces plain peer loads and stores (used by the failure-detection tests).
"""
from __future__ import annotations

import ctypes as C
import heapq
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import LAUNCHES

_BACKENDS: dict = {}
GUARD, GUARD_BYTE = 4096, 0xA5        # guard bands between the regions of a symmetric workspace
DEFAULT_BYTES = int(os.environ.get("NEOX_SYMM_BYTES", 768 * 1024 * 1024))


def _declare():
    L = _lib.lib()
    if getattr(L, "_comm_declared", False):
        return L
    P, I, LL, U, ULL = C.c_void_p, C.c_int, C.c_longlong, C.c_uint, C.c_ulonglong
    PP = C.POINTER(C.c_ulonglong)
    gemm_comm = [P, P, P, I, I, I, LL, LL, LL, I, P, P, P, P, LL, I, I, I, I, U, PP, PP, P, LL, P, LL, P]
    sigs = {"nx_comm_flag_bytes": [], "nx_comm_allreduce": [PP, ULL, I, I, LL, LL, I, U, P],
            "nx_comm_reduce_scatter": [PP, ULL, I, I, LL, LL, P, I, U, P],
            "nx_comm_allgather": [PP, ULL, I, I, LL, LL, P, U, P],
            "nx_gemm_bf16_comm": gemm_comm, "nx_gemm2_bf16_comm": gemm_comm,
            "nx_gemm2_bf16_allreduce": [P, P, I, I, I, LL, LL, I, P, P, LL, I, I, I, U, PP, PP, PP, PP, U, P],
            "nx_gemm_grid": [I, I],
            "nx_comm_zero_reduce_scatter": [PP, I, I, LL, LL, I, I, U, P],
            "nx_comm_embed_push": [PP, I, I, LL, P, P, I, I, I, LL, LL, I, I, U, P],
            "nx_comm_zero_reduce_range": [PP, I, I, LL, LL, LL, LL, I, I, I, U, P],
            "nx_comm_zero_all_gather": [PP, I, I, LL, LL, I, U, P]}
    for name, argtypes in sigs.items():
        for nm in (name, name + "_f16"):            # the bf16 build and the fp16 build of every entry point
            fn = getattr(L, nm)
            fn.argtypes, fn.restype = argtypes, I
    L._comm_declared = True
    return L


class SlotPool:
    """Which of ``n`` equal slots are free.  Every rank of a group makes the same alloc / release / reset calls in the
    same order, so all ranks pick the same slot without talking to each other: ``alloc`` always takes the lowest free
    index."""

    def __init__(self, n: int):
        self.n = int(n)
        self.free = list(range(self.n))
        heapq.heapify(self.free)

    def alloc(self):
        return heapq.heappop(self.free) if self.free else None

    def release(self, slot: int):
        if not 0 <= slot < self.n or slot in self.free:
            raise ValueError(f"slot {slot} is not an allocated slot of this pool")
        heapq.heappush(self.free, slot)

    def reset(self):
        self.free = list(range(self.n))


class SymmBackend:
    def __init__(self, group, nbytes: int = DEFAULT_BYTES):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.ws = dist.get_world_size(group)
        self.me = dist.get_rank(group)
        L = _declare()
        self.flag_bytes = L.nx_comm_flag_bytes()
        self.nbytes = nbytes
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.ptrs = (C.c_ulonglong * 8)(*([int(p) for p in self.hdl.buffer_ptrs] + [0] * (8 - self.ws)))
        use_nvls = os.environ.get("NEOX_NVLS", "1") != "0"
        mc = 0
        try:
            if use_nvls and self.hdl.has_multicast_support(dev.type, dev.index):
                mc = int(self.hdl.multicast_ptr)
        except Exception:
            mc = 0
        self.mc = mc
        self.epoch = 1
        # regions: [barrier flags 64K][RS flags 1M][AG flags 16K][collective payload][gather x2][stage x2]; every
        # data region is followed by a guard band of GUARD bytes holding a fixed pattern (check_guards)
        self.rs_flag_off = self.flag_bytes
        self.ag_flag_off = self.rs_flag_off + (1 << 20)
        data0 = self.ag_flag_off + (16 << 10)
        pitch = ((nbytes - data0) // 5) // 4096 * 4096
        unit = pitch - GUARD
        self.unit = unit
        self.payload_bytes = unit
        self.payload = self.buf[self.flag_bytes:]          # collectives address their payload from here
        self.coll_off = data0
        self.gather_off = [data0 + pitch, data0 + 2 * pitch]
        self.stage_off = [data0 + 3 * pitch, data0 + 4 * pitch]
        self.guard_offs = [data0 + i * pitch + unit for i in range(5)]
        for o in self.guard_offs:
            self.buf[o:o + GUARD].fill_(GUARD_BYTE)
        _lib.register_workspace(int(self.hdl.buffer_ptrs[self.me]), nbytes)
        jitter = int(os.environ.get("NEOX_COMM_JITTER_NS", "0"))
        if jitter > 0:
            _lib.set_comm_jitter_ns(jitter)
        self.ag_calls = 0
        self.rs_calls = 0
        self.ar_calls = 0
        self.pool = None                                      # gather-buffer pool: created by the first keep=True gather
        self.ar_count_off = self.ag_flag_off + (8 << 10)      # upper half of the all-gather flag area
        self.ar_target = 0
        dist.barrier(group)

    def check_guards(self) -> bool:
        """True if no kernel wrote past the end of a data region (synchronises)."""
        torch.cuda.synchronize()
        return all(bool((self.buf[o:o + GUARD] == GUARD_BYTE).all()) for o in self.guard_offs)

    def _table(self, off):
        return (C.c_ulonglong * 8)(*([int(p) + off for p in self.hdl.buffer_ptrs] + [0] * (8 - self.ws)))

    # ------------------------------------------------------------------ fused GEMM + collective
    def can_fuse(self, m_full: int, k: int, n: int) -> bool:
        """Row count divisible into ws chunks of whole 128-row tiles, operands fit the regions."""
        return (m_full % (self.ws * 128) == 0 and k % 8 == 0 and n % 8 == 0 and m_full * k * 2 <= self.unit
                and m_full * n * 2 <= self.unit and (m_full // self.ws // 128) * ((n + 255) // 256) * self.ws * 16
                <= (1 << 20))

    # ------------------------------------------------------------------ pool of gather buffers that outlive a call
    def _pool_create(self, slot_bytes: int):
        """A second symmetric allocation, cut into equal slots: a gathered activation that the backward pass needs
        again (the weight-gradient GEMM) stays where the peers pushed it instead of being copied out of the
        two-deep gather ring.  Collective over the group (first ``ag_gemm(keep=True)``); every rank takes the same
        decision.  NEOX_AG_POOL_GB sizes it (default 8, 0 = off)."""
        import torch.distributed._symmetric_memory as symm_mem
        self.pool = False
        budget = int(float(os.environ.get("NEOX_AG_POOL_GB", "8")) * (1 << 30))
        slot = (slot_bytes + 4095) // 4096 * 4096
        n = min(budget // slot, 512) if slot > 0 else 0          # (small models: do not turn the whole budget into slots)
        ok, buf, hdl = 1, None, None
        if n < 2:
            ok = 0
        else:
            try:
                buf = symm_mem.empty(n * slot, dtype=torch.uint8, device=self.buf.device)
                hdl = symm_mem.rendezvous(buf, self.group)
            except Exception as e:  # noqa: BLE001 - any failure means "keep copying", decided collectively
                print(f"gather-buffer pool unavailable ({type(e).__name__}: {e}); gathered activations are copied", flush=True)
                ok = 0
        flag = torch.tensor([ok], device=self.buf.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            self.pool = {"buf": buf, "hdl": hdl, "slot": slot, "n": n, "slots": SlotPool(n),
                         "ptrs": [int(p) for p in hdl.buffer_ptrs]}

    def pool_alloc(self, nbytes: int):
        """Lowest free slot that holds ``nbytes``, or None (pool off, exhausted, or slots too small).  Every rank of the
        group calls alloc / release / reset at the same points of the program, so all pick the same slot."""
        if self.pool is None:
            self._pool_create(nbytes)
        if not self.pool or nbytes > self.pool["slot"]:
            return None
        return self.pool["slots"].alloc()

    def pool_release(self, slot):
        if slot is not None and self.pool and slot not in self.pool["slots"].free:    # (a reset may have freed it already)
            self.pool["slots"].release(slot)

    def pool_reset(self):
        """Every slot free again (between optimizer steps no gathered activation is alive)."""
        if self.pool:
            self.pool["slots"].reset()

    def ag_gemm(self, x_shard, w, *, trans_b=False, bias=None, gelu=None, aux_out=None, dgelu_aux=None,
                dgelu=None, aux_deriv=False, keep=None):
        """``y = all_gather_rows(x_shard) @ op(w) (+ epilogue)``. Returns (y [M, N], gathered x [M, K]): the
        gathered matrix is a view of the symmetric gather buffer, valid until the second next call.  With
        ``keep`` given (True or False) a third value is returned: a pool slot, or None if none was asked for (False) or
        to be had; with a slot the gathered matrix lives in it until ``pool_release(slot)``.  A peer may push the next gather into a released slot as soon
        as it has finished the fused call that follows the release in program order, so every read of the slot must be
        enqueued BEFORE the first fused call after the release."""
        from ..ops import gemm as G
        ms, k = x_shard.shape
        m = ms * self.ws
        n = w.shape[1] if trans_b else w.shape[0]
        slot = self.pool_alloc(m * k * 2) if keep else None
        if slot is not None:
            so = slot * self.pool["slot"]
            gathered = self.pool["buf"][so:so + m * k * 2].view(x_shard.dtype).view(m, k)
            dst_table = (C.c_ulonglong * 8)(*([p + so for p in self.pool["ptrs"]] + [0] * (8 - self.ws)))
        else:
            par = self.ag_calls & 1
            self.ag_calls += 1
            goff = self.gather_off[par]
            gathered = self.buf[goff:goff + m * k * 2].view(x_shard.dtype).view(m, k)
            dst_table = self._table(goff)
        out = torch.empty((m, n), device=x_shard.device, dtype=x_shard.dtype)
        flags = 0
        ld_aux = 0
        if bias is not None:
            flags |= G.EPI_BIAS
        if gelu is not None:
            flags |= G.EPI_GELU_TANH if gelu == "tanh" else G.EPI_GELU_ERF
        flags |= G.aux_flags(gelu, aux_out, aux_deriv, dgelu_aux, dgelu)
        if aux_out is not None:
            ld_aux = aux_out.stride(0)
        if dgelu_aux is not None:
            ld_aux = dgelu_aux.stride(0)
        epoch = self._next_epoch(1)
        LAUNCHES["n"] += 1
        _lib.check(self._comm_gemm(m, x_shard)(
            _lib.ptr(gathered), _lib.ptr(w), _lib.ptr(out), m, n, k, k, w.stride(0), out.stride(0), int(trans_b),
            _lib.ptr(bias), _lib.ptr(dgelu_aux), _lib.ptr(aux_out), None, ld_aux, flags, 2, self.me, self.ws, epoch,
            dst_table, self._table(self.ag_flag_off), None, 0, _lib.ptr(x_shard), x_shard.stride(0),
            _lib.stream()), "nx_gemm_bf16_comm(all-gather)")
        return (out, gathered, slot) if keep is not None else (out, gathered)

    def gemm_rs(self, a, w, *, trans_b=False, residual=None, bias=None, residual2=None, dgelu_aux=None, dgelu=None):
        """``out = reduce_scatter_rows(a @ op(w) + residual) + bias + residual2`` -> [M / ws, N]."""
        from ..ops import gemm as G
        m, k = a.shape
        n = w.shape[1] if trans_b else w.shape[0]
        par = self.rs_calls & 1
        self.rs_calls += 1
        out = torch.empty((m // self.ws, n), device=a.device, dtype=a.dtype)
        flags = 0
        ld_aux = 0
        if bias is not None:
            flags |= G.EPI_BIAS
        if residual is not None:
            flags |= G.EPI_RESIDUAL
            ld_aux = residual.stride(0)
        if dgelu_aux is not None:
            flags |= G.EPI_DGELU_TANH if dgelu == "tanh" else G.EPI_DGELU_ERF
            assert ld_aux in (0, dgelu_aux.stride(0))
            ld_aux = dgelu_aux.stride(0)
        epoch = self._next_epoch(1)
        LAUNCHES["n"] += 1
        _lib.check(self._comm_gemm(m, a)(
            _lib.ptr(a), _lib.ptr(w), _lib.ptr(out), m, n, k, a.stride(0), w.stride(0), out.stride(0), int(trans_b),
            _lib.ptr(bias), _lib.ptr(dgelu_aux), None, _lib.ptr(residual), ld_aux, flags, 1, self.me, self.ws, epoch,
            self._table(self.stage_off[par]), self._table(self.rs_flag_off), _lib.ptr(residual2),
            residual2.stride(0) if residual2 is not None else 0, None, 0, _lib.stream()),
            "nx_gemm_bf16_comm(reduce-scatter)")
        return out

    def can_fuse_ar(self, m: int, k: int, n: int) -> bool:
        from ..ops.gemm import PAIR_GEMM
        if os.environ.get("NEOX_FUSED_AR", "1") == "0":
            return False
        return bool(PAIR_GEMM["on"]) and m % (self.ws * 256) == 0 and self.can_fuse(m, k, n)

    def gemm_ar(self, a, w, *, trans_b=False, bias=None, residual=None):
        """``out = all_reduce(a @ op(w) + residual) + bias`` -> [M, N], every rank gets the full result.
        Reduce-scatter inside the GEMM epilogue, then each owner stores its reduced rows into every rank's
        output; the result is a view of the symmetric workspace, valid until the second next call."""
        from ..ops import gemm as G
        m, k = a.shape
        n = w.shape[1] if trans_b else w.shape[0]
        par = self.ar_calls & 1
        self.ar_calls += 1
        ooff = self.gather_off[par]
        out = self.buf[ooff:ooff + m * n * 2].view(a.dtype).view(m, n)
        flags, ld_aux = 0, 0
        if bias is not None:
            flags |= G.EPI_BIAS
        if residual is not None:
            flags |= G.EPI_RESIDUAL
            ld_aux = residual.stride(0)
        tiles = (m // self.ws // 256) * ((n + 255) // 256)
        self.ar_target = (self.ar_target + (self.ws - 1) * tiles * 8) & 0xFFFFFFFF
        epoch = self._next_epoch(1)
        LAUNCHES["n"] += 2
        _lib.check(_lib.lib(a).nx_gemm2_bf16_allreduce(
            _lib.ptr(a), _lib.ptr(w), m, n, k, a.stride(0), w.stride(0), int(trans_b), _lib.ptr(bias),
            _lib.ptr(residual), ld_aux, flags, self.me, self.ws, epoch, self._table(self.stage_off[par]),
            self._table(self.rs_flag_off), self._table(ooff), self._table(self.ar_count_off), self.ar_target,
            _lib.stream()), "nx_gemm2_bf16_allreduce")
        return out

    def _comm_gemm(self, m_full: int, like):
        """CTA-pair kernel (256-row tiles) when the rank chunks are whole 256-row tiles, else the 128-row kernel;
        the bf16 or the fp16 build by the dtype of ``like``."""
        from ..ops.gemm import PAIR_GEMM
        L = _lib.lib(like)
        return L.nx_gemm2_bf16_comm if (PAIR_GEMM["on"] and m_full % (self.ws * 256) == 0) else L.nx_gemm_bf16_comm

    def supports(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and x.is_contiguous()
                and (x.numel() * x.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0)

    def _next_epoch(self, n=2):
        e = self.epoch
        self.epoch += n
        return e

    def _view(self, nbytes, dtype, shape):
        return self.buf[self.coll_off:self.coll_off + nbytes].view(dtype).view(shape)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        nb = x.numel() * x.element_size()
        if nb > self.payload_bytes:
            dist.all_reduce(x, group=self.group)
            return x
        stage = self._view(nb, x.dtype, x.shape)
        stage.copy_(x)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x).nx_comm_allreduce(self.ptrs, self.mc, self.me, self.ws, self.coll_off, nb,
                                                1 if x.dtype == torch.float32 else 0, self._next_epoch(),
                                                _lib.stream()), "nx_comm_allreduce")
        x.copy_(stage)
        return x

    def can_embed_push(self, ids: torch.Tensor, table: torch.Tensor, sp: bool) -> bool:
        b, s = ids.shape
        rows = b * (s // self.ws if sp else s)
        return (ids.dim() == 2 and ids.dtype == torch.int64 and table.dtype in _lib.H16 and table.shape[1] % 8 == 0
                and (not sp or s % self.ws == 0) and rows * table.shape[1] * 2 <= self.payload_bytes)

    def embed_push(self, ids: torch.Tensor, table: torch.Tensor, vocab_lo: int, sp: bool) -> torch.Tensor:
        """Vocabulary-parallel embedding of ``ids`` [B, S] without a reduction: every rank stores the rows of the ids
        it owns straight into the output of the ranks that need them.  Returns [B, S, H], or this rank's
        [B, S / ws, H] slice along the sequence with ``sp``."""
        b, s = ids.shape
        h = table.shape[1]
        s_loc = s // self.ws if sp else s
        LAUNCHES["n"] += 1
        grid = min(2 * torch.cuda.get_device_properties(ids.device).multi_processor_count, 1024)
        _lib.check(_lib.lib(table).nx_comm_embed_push(self.ptrs, self.me, self.ws, self.coll_off,
                                                      _lib.ptr(ids.contiguous()), _lib.ptr(table), b, s, h, int(vocab_lo),
                                                      table.shape[0], 1 if sp else 0, grid, self._next_epoch(),
                                                      _lib.stream()), "nx_comm_embed_push")
        return self._view(b * s_loc * h * 2, table.dtype, (b, s_loc, h)).clone()

    def reduce_scatter0(self, x: torch.Tensor) -> torch.Tensor:
        nb = x.numel() * x.element_size()
        shard = nb // self.ws
        if nb > self.payload_bytes or shard % 16 or x.shape[0] % self.ws:
            out = torch.empty((x.shape[0] // self.ws,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, x, group=self.group)
            return out
        self._view(nb, x.dtype, x.shape).copy_(x)
        out = torch.empty((x.shape[0] // self.ws,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(x).nx_comm_reduce_scatter(self.ptrs, self.mc, self.me, self.ws, self.coll_off, shard, _lib.ptr(out),
                                                     1 if x.dtype == torch.float32 else 0, self._next_epoch(),
                                                     _lib.stream()), "nx_comm_reduce_scatter")
        return out

    def all_gather0(self, x: torch.Tensor) -> torch.Tensor:
        shard = x.numel() * x.element_size()
        nb = shard * self.ws
        if nb > self.payload_bytes:
            out = torch.empty((self.ws * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(out, x, group=self.group)
            return out
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib().nx_comm_allgather(self.ptrs, self.mc, self.me, self.ws, self.coll_off, shard, _lib.ptr(x),
                                                self._next_epoch(), _lib.stream()), "nx_comm_allgather")
        return self._view(nb, x.dtype, (self.ws * x.shape[0],) + tuple(x.shape[1:])).clone()


def init_group(group, nbytes: int = DEFAULT_BYTES):
    """Create (once) the symmetric workspace of ``group``. Collective: every rank of the group calls it."""
    key = id(group) if group is not None else 0
    if key not in _BACKENDS:
        _BACKENDS[key] = SymmBackend(group, nbytes)
    return _BACKENDS[key]


def backend_for(group):
    return _BACKENDS.get(id(group) if group is not None else 0)


def reset():
    _BACKENDS.clear()


def pool_reset_all():
    """Free every slot of every group's gather-buffer pool (the engine calls this between optimizer steps)."""
    for be in _BACKENDS.values():
        be.pool_reset()


class ZeroWorkspace:
    """Symmetric home of one flat parameter space's gradient and low-precision parameter buffers, so the
    ZeRO reduce-scatter and all-gather run in place over peer memory (csrc/comm.cu, zero_* kernels):
    no staging copies and no NCCL on the optimizer step.  Layout: [flags 64 KiB][gradients][parameters]."""

    def __init__(self, group, grad_bytes: int, param_bytes: int):
        import torch.distributed._symmetric_memory as symm_mem
        L = _declare()
        P, I, LL, U = C.c_void_p, C.c_int, C.c_longlong, C.c_uint
        PP = C.POINTER(C.c_ulonglong)
        self.group, self.ws, self.me = group, dist.get_world_size(group), dist.get_rank(group)
        self.flag_bytes = L.nx_comm_flag_bytes()
        al = lambda n: (n + 4095) // 4096 * 4096 + GUARD       # each buffer is followed by a guard band
        self.grad_off = self.flag_bytes
        self.param_off = self.grad_off + al(grad_bytes)
        total = self.param_off + al(param_bytes)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.buf[: self.flag_bytes].zero_()
        torch.cuda.synchronize()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.ptrs = (C.c_ulonglong * 8)(*([int(p) for p in self.hdl.buffer_ptrs] + [0] * (8 - self.ws)))
        self.grad_bytes, self.param_bytes = grad_bytes, param_bytes
        self.guard_offs = [self.param_off - GUARD, total - GUARD]
        for o in self.guard_offs:
            self.buf[o:o + GUARD].fill_(GUARD_BYTE)
        _lib.register_workspace(int(self.hdl.buffer_ptrs[self.me]), total)
        self.epoch = 1
        self.grid = min(2 * torch.cuda.get_device_properties(dev).multi_processor_count, 1024)
        dist.barrier(group)

    def check_guards(self) -> bool:
        torch.cuda.synchronize()
        return all(bool((self.buf[o:o + GUARD] == GUARD_BYTE).all()) for o in self.guard_offs)

    def grad_buffer(self, dtype):
        return self.buf[self.grad_off:self.grad_off + self.grad_bytes].view(dtype)

    def param_buffer(self, dtype):
        return self.buf[self.param_off:self.param_off + self.param_bytes].view(dtype)

    def _next(self):
        e = self.epoch
        self.epoch += 2
        return e

    def reduce_scatter_grads(self, dtype):
        """Sum the gradient buffers of all ranks; rank r ends up with the sum in its chunk r (in place)."""
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(dtype).nx_comm_zero_reduce_scatter(self.ptrs, self.me, self.ws, self.grad_off,
                                                          self.grad_bytes // self.ws,
                                                          1 if dtype == torch.float32 else 0, self.grid, self._next(),
                                                          _lib.stream()), "nx_comm_zero_reduce_scatter")

    #: launch shape of one overlapped bucket reduction: 128-thread blocks need about 10K registers, which is what the
    #: persistent GEMM CTAs of the backward pass leave free on an SM, so the reduction runs beside them; one block per
    #: SM x 4 vectors in flight per thread (1.2 MB) covers the NVLink latency
    RANGE_GRID, RANGE_THREADS = 148, 128

    def reduce_grad_range(self, dtype, lo_bytes: int, hi_bytes: int, stream=None):
        """Sum bytes [lo, hi) of the gradient buffers of all ranks; every part of the range ends up, reduced, in the
        buffer of the rank whose chunk it belongs to.  Every rank calls this with the same ranges in the same order."""
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib(dtype).nx_comm_zero_reduce_range(self.ptrs, self.me, self.ws, self.grad_off,
                                                             self.grad_bytes // self.ws, lo_bytes, hi_bytes,
                                                             1 if dtype == torch.float32 else 0, self.RANGE_GRID,
                                                             self.RANGE_THREADS, self._next(), stream if stream is not None else _lib.stream()),
                   "nx_comm_zero_reduce_range")

    def all_gather_params(self):
        """Push this rank's chunk of the parameter buffer into every peer's buffer (in place)."""
        LAUNCHES["n"] += 1
        _lib.check(_lib.lib().nx_comm_zero_all_gather(self.ptrs, self.me, self.ws, self.param_off,
                                                      self.param_bytes // self.ws, self.grid, self._next(),
                                                      _lib.stream()), "nx_comm_zero_all_gather")
