"""Training engine: what the reference obtains from ``deepspeed.initialize`` (megatron/training.py:1188-1198):
mixed precision with fp32 master weights, gradient accumulation, ZeRO-1/2 optimizer-state
partitioning over the data-parallel group, global-norm clipping, fp16 dynamic loss scaling, the
optimizer step and the learning-rate schedule.

Layout (designed for 180 GB of HBM per GPU and NVSwitch collectives, not ported from DeepSpeed):
every parameter of a data-parallel group lives in ONE flat low-precision buffer, ordered
[decay | no-decay] x [tensor-parallel-sharded | replicated]; a flat fp32 ``main_grad`` buffer of the
same shape receives gradients (GEMM weight gradients are accumulated straight into it by the wgrad
epilogue).  At the accumulation boundary the flat gradient is reduce-scattered once, each rank runs
the fused AdamW kernel on its contiguous shard (fp32 master + moments, clip / unscale factor read
from device memory, bf16 weights written in the same pass) and the flat weight buffer is
all-gathered once.  No per-parameter launches, no host synchronisation in bf16 mode.
"""
from __future__ import annotations

import contextlib
import math
import os
from contextlib import contextmanager

import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..ops import optim as optim_ops
from .loss_scaler import LossScaler, build_loss_scaler

_ALIGN = 64  # elements: keeps every parameter 128-byte aligned inside the flat buffer (TMA needs 16)


def _lr_mult(p) -> float:
    """Per-parameter learning-rate multiplier (muP: 1 / width_mult for matrix-like weights under Adam)."""
    return float(getattr(p, "lr_mult", 1.0))


def _is_replicated(p) -> bool:
    """True for parameters that hold the same values on every tensor-parallel rank."""
    return not getattr(p, "model_parallel", False)


def _unit_params(u):
    """Parameters a layer of the stack touches: its own and, for a function layer bound to another layer's module
    (the tied read-out is ``Lambda(partial(fn, embedding))``), that module's."""
    ps = list(u.parameters())
    fn = getattr(u, "func", None)
    for a_ in list(getattr(fn, "args", ())) + list((getattr(fn, "keywords", None) or {}).values()):
        if isinstance(a_, torch.nn.Module):
            ps += [p for p in a_.parameters() if all(p is not q for q in ps)]
    return ps


class FlatGroup:
    """One flat parameter space reduced over one data-parallel process group."""

    def __init__(self, entries, dp_group, dp_size, dp_rank, zero_stage, grad_dtype, state_bits=32,
                 partition_params=False, offload=None):
        # entries: list of (param, weight_decay)
        self.dp_group, self.dp_size, self.dp_rank = dp_group, dp_size, dp_rank
        self.zero_stage = zero_stage
        order = sorted(range(len(entries)), key=lambda i: (0 if entries[i][1] > 0 else 1, entries[i][1],
                                                            1 if _is_replicated(entries[i][0]) else 0,
                                                            1 if getattr(entries[i][0], "_norm_skip", False) else 0,
                                                            _lr_mult(entries[i][0])))
        self.params = [entries[i][0] for i in order]
        self.wds = [entries[i][1] for i in order]
        self.device = self.params[0].device
        self.lp_dtype = self.params[0].dtype
        offs, off = [], 0
        for p in self.params:
            offs.append(off)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        unit = dp_size * 256
        self.total = (off + unit - 1) // unit * unit
        self.offsets = offs
        # (stage 3 allocates and frees the full buffers per module: they cannot live in one symmetric allocation)
        self.zero_ws = None if partition_params else self._try_symmetric_workspace(grad_dtype)
        if self.zero_ws is not None:
            self.flat_lp = self.zero_ws.param_buffer(self.lp_dtype).zero_()
            self.main_grad = self.zero_ws.grad_buffer(grad_dtype).zero_()
        else:
            self.flat_lp = torch.zeros(self.total, dtype=self.lp_dtype, device=self.device)
            self.main_grad = torch.zeros(self.total, dtype=grad_dtype, device=self.device)
        for p, o in zip(self.params, offs):
            n = p.numel()
            self.flat_lp[o:o + n].copy_(p.data.reshape(-1))
            p.data = self.flat_lp[o:o + n].view(p.shape)
            p.main_grad = self.main_grad[o:o + n].view(p.shape)
            p.grad = None
        # regions of constant (weight decay, replicated, norm-skip, learning-rate multiplier)
        self.regions = []
        for p, o, wd in zip(self.params, offs, self.wds):
            key = (wd, _is_replicated(p), bool(getattr(p, "_norm_skip", False)), _lr_mult(p))
            end = o + (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
            if self.regions and self.regions[-1][2:] == key and self.regions[-1][1] == o:
                self.regions[-1] = (self.regions[-1][0], end) + key
            else:
                self.regions.append((o, end) + key)
        sharded = zero_stage >= 1 and dp_size > 1
        self.shard_size = self.total // dp_size if sharded else self.total
        self.shard_start = dp_rank * self.shard_size if sharded else 0
        self.sharded = sharded
        s, e = self.shard_start, self.shard_start + self.shard_size
        if self.lp_dtype == torch.float32:
            self.master = self.flat_lp[s:e]
        else:
            self.master = self.flat_lp[s:e].float()
        # Adam moments of the shard: fp32, or (``use_bnb_optimizer``) one byte per element with one fp32 scale per
        # 2048 elements of every segment (ops/optim.py adamw8bit_step_)
        self.state_bits = state_bits
        state_dtype = torch.float32 if state_bits == 32 else torch.uint8
        self.exp_avg = torch.zeros(self.shard_size, dtype=state_dtype, device=self.device)
        self.exp_avg_sq = torch.zeros(self.shard_size, dtype=state_dtype, device=self.device)
        # my shard's intersections with the regions: (lo, hi, wd, replicated, norm_skip, lr_mult), shard-relative
        self.segments = []
        for (a, b, wd, rep, skip, lrm) in self.regions:
            lo, hi = max(a, s), min(b, e)
            if hi > lo:
                self.segments.append((lo - s, hi - s, wd, rep, skip, lrm))
        # ZeRO stage 3: between uses only this rank's slice of the parameters (and of the gradients) is kept
        self.partition_params = bool(partition_params) and sharded
        self.grad_dtype = grad_dtype
        self.shapes = [tuple(p.shape) for p in self.params]
        self.lp_shard = None
        self.grad_acc = None
        if self.partition_params:
            self.lp_shard = self.flat_lp[s:e].clone()
            if self.lp_dtype == torch.float32:
                self.master = self.lp_shard          # fp32 parameters are their own master weights
            self.grad_acc = torch.zeros(self.shard_size, dtype=grad_dtype, device=self.device)
            self.release()
        # optimizer-state offload: master weights and moments of the shard in (pinned) host memory, plus staging
        # buffers for the gradient shard on its way down and the new 16-bit weights on their way up
        self.offload = offload if (offload and state_bits == 32) else None
        if self.offload:
            pin = self.device.type == "cuda"
            host = lambda t: t.detach().to("cpu", copy=True).pin_memory() if pin else t.detach().to("cpu", copy=True)   # noqa: E731
            self.master = host(self.master.float())
            self.exp_avg, self.exp_avg_sq = host(self.exp_avg), host(self.exp_avg_sq)
            self.host_grad = host(torch.zeros(self.shard_size, dtype=grad_dtype))
            self.host_lp = host(torch.zeros(self.shard_size, dtype=self.lp_dtype))
        # bucketed gradient reduction overlapped with the backward pass (Engine._ov_*): element ranges already
        # reduced (or in flight) this step, outstanding collective handles, the stream the peer-memory kernels run on
        self._reduced, self._works, self._side = [], [], None
        self.q8_scales = None
        if state_bits == 8:
            self.q8_scales = [torch.zeros((2, optim_ops.q8_blocks(hi - lo)), dtype=torch.float32, device=self.device)
                              for (lo, hi, *_rest) in self.segments]

    def _try_symmetric_workspace(self, grad_dtype):
        """ZeRO over peer memory: put the gradient and parameter buffers into a symmetric allocation of the
        data-parallel group so the reduce-scatter / all-gather kernels work on them in place.  Every rank of
        the group takes the same decision (the attempt's outcome is min-reduced)."""
        import os
        from ..comm import collectives
        if not (self.device.type == "cuda" and self.dp_size > 1 and self.zero_stage >= 1
                and collectives.get_mode() == "fused" and os.environ.get("NEOX_ZERO_SYMM", "1") != "0"
                and grad_dtype in (torch.float32, torch.bfloat16, torch.float16) and self.dp_size <= 8):
            return None
        ws, ok = None, 1
        try:
            from ..comm.symm import ZeroWorkspace
            esz = lambda dt: torch.empty((), dtype=dt).element_size()
            ws = ZeroWorkspace(self.dp_group, self.total * esz(grad_dtype), self.total * esz(self.lp_dtype))
        except Exception as e:  # noqa: BLE001 - any failure means "use the NCCL path", decided collectively
            print(f"ZeRO symmetric workspace unavailable ({type(e).__name__}: {e}); using NCCL collectives", flush=True)
            ok = 0
        flag = torch.tensor([ok], device=self.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.dp_group)
        return ws if int(flag.item()) == 1 else None

    def numel(self):
        return sum(math.prod(sh) for sh in self.shapes)

    # ------------------------------------------------------------------ ZeRO stage 3: gather / release
    @property
    def gathered(self):
        return self.flat_lp is not None

    def gather(self, with_grads=False):
        """Materialise the whole flat parameter buffer from the ranks' slices (all-gather) and point the
        parameters into it; ``with_grads`` also provides the full-size gradient buffer a backward pass writes."""
        if not self.partition_params:
            return
        if self.flat_lp is None:
            self.flat_lp = torch.empty(self.total, dtype=self.lp_dtype, device=self.device)
            if self.flat_lp.is_cuda:
                dist.all_gather_into_tensor(self.flat_lp, self.lp_shard, group=self.dp_group)
            else:
                parts = [torch.empty_like(self.lp_shard) for _ in range(self.dp_size)]
                dist.all_gather(parts, self.lp_shard, group=self.dp_group)
                self.flat_lp.copy_(torch.cat(parts))
            for p, o, sh in zip(self.params, self.offsets, self.shapes):
                p.data = self.flat_lp[o:o + math.prod(sh)].view(sh)
        if with_grads and self.main_grad is None:
            self.main_grad = torch.zeros(self.total, dtype=self.grad_dtype, device=self.device)
            for p, o, sh in zip(self.params, self.offsets, self.shapes):
                p.main_grad = self.main_grad[o:o + math.prod(sh)].view(sh)

    def release(self):
        """Drop the gathered buffers; the parameters keep their identity but hold no storage until the next gather."""
        if not self.partition_params:
            return
        for p in self.params:
            p.data = torch.empty(0, dtype=self.lp_dtype, device=self.device)
            p.main_grad = None
        self.flat_lp = None
        self.main_grad = None

    def finish_backward(self):
        """After the backward pass of the modules that own these parameters: reduce-scatter the full gradient
        buffer of this micro-batch into the rank's persistent gradient slice, then release everything."""
        if not self.partition_params or self.main_grad is None:
            return
        self.fold_autograd_grads()
        if self.predivide != 1.0:
            self.main_grad.mul_(1.0 / self.predivide)
        part = torch.empty(self.shard_size, dtype=self.grad_dtype, device=self.device)
        if self.main_grad.is_cuda:
            dist.reduce_scatter_tensor(part, self.main_grad, group=self.dp_group)
        else:
            dist.all_reduce(self.main_grad, group=self.dp_group)
            part.copy_(self.main_grad[self.shard_start:self.shard_start + self.shard_size])
        self.grad_acc.add_(part)
        self.release()

    def store_shard_from_gathered(self):
        """Take this rank's slice of the (modified) gathered parameters as the new persistent slice."""
        if self.partition_params and self.flat_lp is not None:
            self.lp_shard.copy_(self.flat_lp[self.shard_start:self.shard_start + self.shard_size])

    def fold_autograd_grads(self):
        """Parameters whose gradient came through plain autograd (``.grad``) are added into
        ``main_grad``; GEMM weights were accumulated there directly by the wgrad epilogue."""
        if self.main_grad is None:
            return
        for p, o in zip(self.params, self.offsets):
            if p.grad is not None:
                if any(lo <= o < hi for lo, hi in self._reduced):
                    raise RuntimeError("a gradient arrived after its bucket was reduced (overlap_comm): a parameter is "
                                       "used by a layer that runs its backward after the layer that owns it")
                p.main_grad.add_(p.grad.view_as(p.main_grad).to(p.main_grad.dtype))
                p.grad = None

    # ------------------------------------------------------------------ bucketed reduction, overlapped with backward
    def param_ranges(self, params):
        """Element ranges [lo, hi) of the flat space that hold ``params`` (padding included), adjacent ones merged."""
        at = {id(p): o for p, o in zip(self.params, self.offsets)}
        spans = sorted((at[id(p)], at[id(p)] + (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN) for p in params if id(p) in at)
        out = []
        for lo, hi in spans:
            if out and out[-1][1] == lo:
                out[-1] = (out[-1][0], hi)
            else:
                out.append((lo, hi))
        return out

    def reduce_range_async(self, lo, hi):
        """Start the data-parallel sum of main_grad[lo:hi] (complete on every rank) without waiting for it: over
        peer memory on a side stream when the buffers are symmetric (each part lands in its owner's buffer), else
        as an asynchronous all-reduce of the range.  ``reduce_gradients`` covers what is left and waits."""
        if hi <= lo:
            return
        self._reduced.append((lo, hi))
        if self.predivide != 1.0:
            self.main_grad[lo:hi].mul_(1.0 / self.predivide)
        if self.dp_size == 1:
            return
        if self.zero_ws is not None:
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.device)
            self._side.wait_stream(torch.cuda.current_stream())
            esz = self.main_grad.element_size()
            with torch.cuda.stream(self._side):
                self.zero_ws.reduce_grad_range(self.main_grad.dtype, lo * esz, hi * esz)
        else:
            self._works.append(dist.all_reduce(self.main_grad[lo:hi], group=self.dp_group, async_op=True))

    def _finish_bucketed(self):
        """Reduce whatever no bucket covered, then wait for every bucket."""
        covered, at = sorted(self._reduced), 0
        for lo, hi in covered + [(self.total, self.total)]:
            if lo > at:
                self.reduce_range_async(at, lo)
            at = max(at, hi)
        if self._side is not None:
            torch.cuda.current_stream().wait_stream(self._side)
        for w in self._works:
            w.wait()
        self._reduced, self._works = [], []

    def grad_shard(self):
        if self.partition_params:
            return self.grad_acc
        return self.main_grad[self.shard_start:self.shard_start + self.shard_size]

    def lp_shard_view(self):
        """This rank's slice of the low-precision parameters (what the optimizer step writes)."""
        if self.partition_params:
            return self.lp_shard
        return self.flat_lp[self.shard_start:self.shard_start + self.shard_size]

    #: gradients are multiplied by 1 / predivide before the reduction (the engine folds the factor back into
    #: its post-reduction scale); comm_dtype, when set, is the dtype the reduction runs in
    predivide = 1.0
    comm_dtype = None

    def reduce_gradients(self):
        if self.partition_params:
            return                # every micro-batch's gradients were reduce-scattered right after its backward
        if self._reduced:
            self._finish_bucketed()   # the layers' buckets were started from the backward pass
            return
        if self.predivide != 1.0:
            self.main_grad.mul_(1.0 / self.predivide)
        if self.dp_size == 1:
            return
        if self.comm_dtype is not None and self.comm_dtype != self.main_grad.dtype:
            # reduce in another precision (``communication_data_type``): one cast each way, plain collectives
            buf = self.main_grad.to(self.comm_dtype)
            dist.all_reduce(buf, group=self.dp_group)
            self.main_grad.copy_(buf)
            return
        if self.zero_ws is not None:
            # reduce-scatter straight out of the peers' gradient buffers, result in place in this rank's shard
            self.zero_ws.reduce_scatter_grads(self.main_grad.dtype)
            return
        if self.sharded:
            out = self.grad_shard()
            if self.main_grad.is_cuda:
                dist.reduce_scatter_tensor(out, self.main_grad, group=self.dp_group)
            else:
                dist.all_reduce(self.main_grad, group=self.dp_group)
        else:
            dist.all_reduce(self.main_grad, group=self.dp_group)

    def gather_params(self):
        if self.partition_params:
            return                # parameters are gathered per module, when its forward / backward needs them
        if self.zero_ws is not None:
            self.zero_ws.all_gather_params()      # push the updated shard into every peer's parameter buffer
            return
        if self.sharded:
            lp_shard = self.flat_lp[self.shard_start:self.shard_start + self.shard_size]
            if self.flat_lp.is_cuda:
                dist.all_gather_into_tensor(self.flat_lp, lp_shard, group=self.dp_group)
            else:
                parts = [torch.empty_like(lp_shard) for _ in range(self.dp_size)]
                dist.all_gather(parts, lp_shard.clone(), group=self.dp_group)
                self.flat_lp.copy_(torch.cat(parts))

    def zero_grad(self):
        if self.partition_params:
            self.grad_acc.zero_()
        if self.main_grad is not None:
            self.main_grad.zero_()
        for p in self.params:
            p.grad = None

    # ------------------------------------------------------------------ checkpoint support
    def shard_state(self):
        return {"master": self.master.detach().clone().cpu() if self.lp_dtype != torch.float32 else
                self.master.detach().clone().cpu(),
                "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
                "q8_scales": None if self.q8_scales is None else [t.cpu() for t in self.q8_scales],
                "shard_start": self.shard_start, "shard_size": self.shard_size, "total": self.total}

    def load_shard_state(self, sd):
        if sd["shard_size"] == self.shard_size and sd["shard_start"] == self.shard_start and \
                sd["exp_avg"].dtype == self.exp_avg.dtype:
            if self.q8_scales is not None:
                saved = sd.get("q8_scales") or []
                if [tuple(t.shape) for t in saved] != [tuple(t.shape) for t in self.q8_scales]:
                    return False
                for dst, src in zip(self.q8_scales, saved):
                    dst.copy_(src)
            self.exp_avg.copy_(sd["exp_avg"])
            self.exp_avg_sq.copy_(sd["exp_avg_sq"])
            if self.lp_dtype != torch.float32 or self.offload:
                self.master.copy_(sd["master"])
            return True
        return False

    def refresh_master_from_lp(self):
        if self.offload:
            self.master.copy_(self.lp_shard_view().float())
            return
        if self.lp_dtype != torch.float32:
            self.master.copy_(self.lp_shard_view().float())
        elif self.partition_params:
            self.master = self.lp_shard


class FlatAdam:
    """Optimizer facade over the flat groups: ``param_groups`` (for the LR schedule and logging),
    ``step``, ``state_dict`` / ``load_state_dict``, ``overflow`` and ``cur_scale`` as the reference
    reads them from its engine's optimizer (megatron/training.py:1380,1518)."""

    def __init__(self, groups, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adam_w_mode=True,
                 generic_cls=None, generic_kwargs=None, state_bits=32):
        self.groups = groups
        self.defaults = {"lr": lr, "betas": tuple(betas), "eps": eps, "weight_decay": weight_decay}
        self.adam_w_mode = adam_w_mode
        self.param_groups = [
            {"params": [p for g in groups for p, wd in zip(g.params, g.wds) if wd > 0], "lr": lr,
             "betas": tuple(betas), "eps": eps, "weight_decay": weight_decay, "name": "weight_decay_params"},
            {"params": [p for g in groups for p, wd in zip(g.params, g.wds) if wd == 0], "lr": lr,
             "betas": tuple(betas), "eps": eps, "weight_decay": 0.0, "name": "no_weight_decay_params"},
        ]
        self.step_count = 0
        self.overflow = False
        self.cur_scale = 1.0
        self.generic = None
        if generic_cls is not None:
            self._seg_params = []
            pgs = []
            for g in groups:
                if not g.sharded:
                    # whole parameters are local: give the optimizer their true shapes (SM3's covers
                    # depend on them); under ZeRO sharding it sees flat 1-D segments, as a flattened
                    # ZeRO partition would present them
                    for p, o, wd in zip(g.params, g.offsets, g.wds):
                        sp = torch.nn.Parameter(g.master[o:o + p.numel()].view(p.shape), requires_grad=True)
                        self._seg_params.append((g, o, o + p.numel(), sp))
                        pgs.append({"params": [sp], "weight_decay": wd, "lr_mult": _lr_mult(p)})
                    continue
                for (lo, hi, wd, _rep, _skip, lrm) in g.segments:
                    sp = torch.nn.Parameter(g.master[lo:hi], requires_grad=True)
                    self._seg_params.append((g, lo, hi, sp))
                    pgs.append({"params": [sp], "weight_decay": wd, "lr_mult": lrm})
            self.generic = generic_cls(pgs, lr=lr, **(generic_kwargs or {}))

    @property
    def lr(self):
        return self.param_groups[0]["lr"]

    def step(self, grad_scale, skip):
        if self.overflow:
            # fp16 overflow, already known on the host: the step is skipped and not counted, so the bias
            # corrections and the saved ``step`` stay those of the updates that really happened
            return
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        b1, b2 = self.param_groups[0]["betas"]
        eps = self.param_groups[0]["eps"]
        if self.generic is not None:
            if skip is not None and int(skip[0]) != 0:
                self.step_count -= 1
                return
            for pg in self.generic.param_groups:
                pg["lr"] = lr * pg.get("lr_mult", 1.0)
            for (g, lo, hi, sp) in self._seg_params:
                sp.grad = (g.grad_shard()[lo:hi].float() * grad_scale[0]).view(sp.shape)
            self.generic.step()
            for g in self.groups:
                if g.lp_dtype != torch.float32:
                    g.flat_lp[g.shard_start:g.shard_start + g.shard_size].copy_(g.master)
            return
        for g in self.groups:
            if g.offload:
                self._offloaded_step(g, lr, b1, b2, eps, grad_scale, skip)
                continue
            gs = g.grad_shard()
            lp_shard = g.lp_shard_view() if g.lp_dtype != torch.float32 else None
            for i, (lo, hi, wd, _rep, _skip, lrm) in enumerate(g.segments):
                if g.state_bits == 8:
                    optim_ops.adamw8bit_step_(g.master[lo:hi], g.exp_avg[lo:hi], g.exp_avg_sq[lo:hi], g.q8_scales[i][0],
                                              g.q8_scales[i][1], gs[lo:hi],
                                              lp_shard[lo:hi] if lp_shard is not None else None, lr=lr * lrm, beta1=b1,
                                              beta2=b2, eps=eps, weight_decay=wd, step=self.step_count,
                                              adam_w_mode=self.adam_w_mode, grad_scale=grad_scale, skip=skip)
                    continue
                optim_ops.adamw_step_(g.master[lo:hi], g.exp_avg[lo:hi], g.exp_avg_sq[lo:hi], gs[lo:hi],
                                      lp_shard[lo:hi] if lp_shard is not None else None,
                                      lr=lr * lrm, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=self.step_count,
                                      adam_w_mode=self.adam_w_mode, grad_scale=grad_scale, skip=skip)

    def _offloaded_step(self, g, lr, b1, b2, eps, grad_scale, skip):
        """Optimizer-state offload: gradient shard to the host, AdamW there, new 16-bit weights back to the device."""
        g.host_grad.copy_(g.grad_shard(), non_blocking=True)
        if g.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        if skip is not None and int(skip[0]) != 0:
            return
        scale = float(grad_scale[0]) if grad_scale is not None else 1.0
        for (lo, hi, wd, _rep, _skip, lrm) in g.segments:
            if g.offload == "native":
                optim_ops.cpu_adamw_step_(g.master[lo:hi], g.exp_avg[lo:hi], g.exp_avg_sq[lo:hi], g.host_grad[lo:hi],
                                          g.host_lp[lo:hi], lr=lr * lrm, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                                          step=self.step_count, adam_w_mode=self.adam_w_mode, grad_scale=scale)
            else:                       # "torch": the same update with PyTorch's CPU operators
                optim_ops.adamw_step_(g.master[lo:hi], g.exp_avg[lo:hi], g.exp_avg_sq[lo:hi], g.host_grad[lo:hi],
                                      g.host_lp[lo:hi], lr=lr * lrm, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                                      step=self.step_count, adam_w_mode=self.adam_w_mode,
                                      grad_scale=torch.tensor([scale]), skip=None)
        g.lp_shard_view().copy_(g.host_lp, non_blocking=True)

    def zero_grad(self, set_to_none=True):
        for g in self.groups:
            g.zero_grad()

    def state_dict(self):
        return {"step": self.step_count, "param_groups": [{k: v for k, v in pg.items() if k != "params"}
                                                           for pg in self.param_groups],
                "shards": [g.shard_state() for g in self.groups], "cur_scale": self.cur_scale,
                # SM3 / MADGRAD / Lion / SGD keep their own per-parameter state (covers, momenta)
                "generic": None if self.generic is None else self.generic.state_dict()}

    def load_state_dict(self, sd):
        self.step_count = sd.get("step", 0)
        for pg, spg in zip(self.param_groups, sd.get("param_groups", [])):
            pg.update({k: v for k, v in spg.items() if k != "params"})
        ok = True
        for g, s in zip(self.groups, sd.get("shards", [])):
            ok = g.load_shard_state(s) and ok
        self.cur_scale = sd.get("cur_scale", self.cur_scale)
        if self.generic is not None and sd.get("generic") is not None:
            try:
                self.generic.load_state_dict(sd["generic"])
            except (ValueError, RuntimeError, KeyError) as e:       # different sharding: its state starts afresh
                print(f"WARNING: state of {type(self.generic).__name__} not restored ({e})", flush=True)
                ok = False
        return ok


class Engine(torch.nn.Module):
    """forward / backward / step with gradient accumulation over the flat groups above."""

    def __init__(self, module, neox_args, param_groups, optimizer_cfg=None, lr_scheduler=None,
                 generic_optimizer=None):
        super().__init__()
        self.module = module
        self.neox_args = neox_args
        a = neox_args
        self.gradient_accumulation_steps = a.gradient_accumulation_steps
        self.micro_steps = 0
        self.global_steps = 0
        self.skipped_steps = 0
        self.global_samples = 0
        self.zero_stage = a.zero_stage if isinstance(a.zero_stage, int) else 0
        if self.zero_stage >= 3 and (mpu.get_model_parallel_world_size() > 1 or a.is_pipe_parallel):
            raise ValueError("ZeRO stage 3 runs with tensor-parallel size 1 and without pipeline parallelism "
                             "(as in the reference, megatron/training.py:878-893)")
        self.gradient_clipping = a.gradient_clipping or 0.0
        self.fp16_enabled = a.precision == "fp16"
        self.bfloat16_enabled = a.precision == "bfloat16"
        self.loss_scaler = build_loss_scaler(a.fp16) if self.fp16_enabled else LossScaler(1.0)
        grad_dtype = torch.float32 if (a.fp32_grad_accum or a.precision == "fp32") else a.params_dtype
        # 8-bit Adam moments when the optimizer configuration asks for them (and the fused Adam path is the optimizer)
        state_bits = int((optimizer_cfg or {}).get("state_bits", 32)) if not generic_optimizer else 32
        offload = (optimizer_cfg or {}).get("offload") if not generic_optimizer else None      # None | "native" | "torch"
        dense, expert = [], []
        for pg in param_groups:
            wd = pg.get("weight_decay", a.weight_decay)
            for p in pg["params"]:
                # muP scales the decay of matrix-like weights by their width multiplier (lr * wd stays fixed)
                (expert if getattr(p, "expert_parallel", False) else dense).append(
                    (p, wd * float(getattr(p, "wd_mult", 1.0))))
        self.groups = []
        # one flat space per (reduction group, parameter dtype): parameters deliberately kept in fp32
        # inside a bf16 model (Mamba's A_log / D) keep their precision
        def by_dtype(entries):
            out = {}
            for e in entries:
                out.setdefault(e[0].dtype, []).append(e)
            return [out[k] for k in sorted(out, key=lambda d: (d != a.params_dtype, str(d)))]

        self._offload = offload
        self._z3_units = []
        if self.zero_stage >= 3 and mpu.get_data_parallel_world_size() > 1:
            # stage 3: one flat space per layer of the stack, so that a layer's parameters can be gathered for
            # its forward / backward and dropped again; a parameter shared by two layers lives with the first
            dense = self._build_stage3_groups(module, dense, by_dtype, grad_dtype, state_bits)
        for ents in by_dtype(dense):
            gd = torch.float32 if ents[0][0].dtype == torch.float32 else grad_dtype
            self.groups.append(FlatGroup(ents, mpu.get_data_parallel_group(), mpu.get_data_parallel_world_size(),
                                         mpu.get_data_parallel_rank(), self.zero_stage, gd, state_bits, offload=offload))
        for ents in by_dtype(expert):
            ep = mpu.get_expert_parallel_world_size()
            gd = torch.float32 if ents[0][0].dtype == torch.float32 else grad_dtype
            self.groups.append(FlatGroup(ents, mpu.get_expert_data_parallel_group(),
                                         mpu.get_data_parallel_world_size() // ep,
                                         mpu.get_data_parallel_rank() // ep, self.zero_stage, gd, state_bits,
                                         offload=offload))
        self.optimizer = None
        if optimizer_cfg is not None and self.groups:
            self.optimizer = FlatAdam(self.groups, **{k: v for k, v in optimizer_cfg.items() if k != "offload"},
                                      **(generic_optimizer or {}))
            self.optimizer.cur_scale = self.loss_scaler.cur_scale
        self.lr_scheduler = lr_scheduler
        dev = self.groups[0].device if self.groups else torch.device("cpu")
        self._acc = torch.zeros(2, dtype=torch.float32, device=dev)
        self._scale = torch.ones(2, dtype=torch.float32, device=dev)
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)
        self._last_grad_norm = None
        self.store_gradients = False
        self.stored_gradients = None
        self.timer_values = None
        self.curriculum_scheduler = None
        self.training_dataloader = None
        # prescale_gradients: the data-parallel average is taken before the reduction instead of after it;
        # gradient_predivide_factor f: divide by f before and by dp / f after (fp16 / bf16 reductions of many
        # ranks stay in range).  communication_data_type: dtype of the gradient reduction.
        f = float(a.gradient_predivide_factor or 1.0)
        if a.prescale_gradients and f == 1.0:
            f = float(max([g.dp_size for g in self.groups] or [1]))
        self._predivide = f if any(g.dp_size > 1 for g in self.groups) else 1.0
        comm = {None: None, "fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16,
                "bfp16": torch.bfloat16}[a.communication_data_type]
        for g in self.groups:
            g.predivide, g.comm_dtype = self._predivide, comm
        # zero_optimization.overlap_comm: reduce each layer's gradients as soon as its backward is done
        self._ov_pending = None
        self._ov_buckets = 0
        zo = a.zero_optimization or {}
        local = hasattr((generic_optimizer or {}).get("generic_cls"), "wants_local_gradients")   # 1-bit Adam
        if (zo.get("overlap_comm") and os.environ.get("NEOX_ZERO_OVERLAP", "1") != "0" and self.zero_stage < 3
                and not a.is_pipe_parallel and comm is None and not local and any(g.dp_size > 1 for g in self.groups)):
            self._install_overlap_hooks(module)
        # engine-side observability switches (all off by default)
        from ..obs import profiling
        self.breakdown = profiling.StepBreakdown(a.steps_per_print, dev) if a.wall_clock_breakdown else None
        self.flops_profiler = profiling.FlopsProfiler.from_args(module, a)
        self.comms_logger = profiling.CommsLogger.from_args(a)
        if self.comms_logger is not None:
            self.comms_logger.install()
        if a.dump_state:
            profiling.dump_state(self)

    # ------------------------------------------------------------------ ZeRO stage 3
    def _build_stage3_groups(self, module, dense, by_dtype, grad_dtype, state_bits):
        """Creates the per-layer flat groups, installs the gather / release hooks and returns the entries that
        belong to no layer (none in the shipped models; they would stay whole as under stage 1)."""
        wd_of = {id(p): wd for p, wd in dense}
        seq = getattr(module, "sequential", None)
        units = list(seq) if seq is not None else [module]
        owner = {}

        unit_params = _unit_params

        for u in units:
            if not isinstance(u, torch.nn.Module):
                continue
            mine = [p for p in unit_params(u) if id(p) in wd_of and id(p) not in owner]
            groups = []
            for ents in by_dtype([(p, wd_of[id(p)]) for p in mine]):
                gd = torch.float32 if ents[0][0].dtype == torch.float32 else grad_dtype
                g = FlatGroup(ents, mpu.get_data_parallel_group(), mpu.get_data_parallel_world_size(),
                              mpu.get_data_parallel_rank(), self.zero_stage, gd, state_bits, partition_params=True,
                              offload=self._offload)
                self.groups.append(g)
                groups.append(g)
                for p in g.params:
                    owner[id(p)] = g
            needs = []
            for p in unit_params(u):
                g = owner.get(id(p))
                if g is not None and g not in needs:
                    needs.append(g)
            if needs:
                self._z3_units.append((u, needs))
                u.register_forward_pre_hook(lambda _m, _a, needs=needs: self._z3_before_forward(needs))
                u.register_forward_hook(lambda _m, _a, _o, needs=needs: self._z3_after_forward(needs))
                u.register_full_backward_pre_hook(lambda _m, _g, needs=needs: self._z3_before_backward(needs))
        self._z3_pending = None
        return [(p, wd) for p, wd in dense if id(p) not in owner]

    def _z3_before_forward(self, needs):
        for g in needs:
            g.gather()

    def _z3_after_forward(self, needs):
        # inside a backward pass (activation recompute) the parameters are needed again at once
        if self._z3_pending is not needs:
            for g in needs:
                if g.main_grad is None:
                    g.release()

    def _z3_before_backward(self, needs):
        """A layer's backward is about to run: the layer whose backward ran before it is complete now (its gradients
        are reduce-scattered and its buffers dropped), and this layer's parameters and gradient buffer are set up."""
        if self._z3_pending is not None and self._z3_pending is not needs:
            for g in self._z3_pending:
                if g not in needs:
                    g.finish_backward()
        for g in needs:
            g.gather(with_grads=True)
        self._z3_pending = needs

    def _z3_finish(self):
        if self._z3_units and self._z3_pending is not None:
            for g in self._z3_pending:
                g.finish_backward()
            self._z3_pending = None
        for g in self.groups:          # parameters shared between layers may still hold a gradient buffer
            if g.partition_params and g.main_grad is not None:
                g.finish_backward()

    # ------------------------------------------------------------------ gradient reduction overlapped with backward
    def _install_overlap_hooks(self, module):
        """One bucket per layer of the stack: the ranges of the flat gradient buffers that hold the parameters the
        layer is the first (in forward order) to use.  On the last micro-batch of a step a layer's bucket is
        reduced when the backward of the next layer down begins: by then every node of its own backward has run
        (autograd runs nodes latest-created first), and a parameter shared with a later layer is complete too,
        since that layer's backward ran earlier.  What DeepSpeed's ``overlap_comm`` does with per-parameter hooks
        and ``reduce_bucket_size`` buckets (reference configs/pythia/1-4B.yml:33), here one launch per layer."""
        seq = getattr(module, "sequential", None)
        where = {id(p): g for g in self.groups for p in g.params if g.dp_size > 1 and not g.partition_params}
        seen = set()
        for u in (list(seq) if seq is not None else []):
            if not isinstance(u, torch.nn.Module):
                continue
            mine = [p for p in _unit_params(u) if id(p) in where and id(p) not in seen]
            seen.update(id(p) for p in mine)
            bucket = []
            for g in self.groups:
                ps = [p for p in mine if where[id(p)] is g]
                if ps:
                    bucket.append((g, ps, g.param_ranges(ps)))
            if bucket:
                self._ov_buckets += 1
                u.register_full_backward_pre_hook(lambda _m, _g, b=bucket: self._ov_before_backward(b))

    def _ov_active(self):
        return self._ov_buckets > 0 and self.is_gradient_accumulation_boundary() and not self.store_gradients

    def _ov_before_backward(self, bucket):
        if not self._ov_active():
            return
        if self._ov_pending is not None and self._ov_pending is not bucket:
            self._ov_launch(self._ov_pending)
        self._ov_pending = bucket

    def _ov_launch(self, bucket):
        for g, params, ranges in bucket:
            for p in params:
                if p.grad is not None:
                    p.main_grad.add_(p.grad.view_as(p.main_grad).to(p.main_grad.dtype))
                    p.grad = None
            for lo, hi in ranges:
                g.reduce_range_async(lo, hi)

    def _ov_finish(self):
        if self._ov_pending is not None:
            self._ov_launch(self._ov_pending)
            self._ov_pending = None

    @contextmanager
    def gathered_parameters(self, write_back=False):
        """All parameters materialised (state dicts, conversions, weight surgery).  ``write_back``: the ranks keep
        their slices of whatever the block wrote into the parameters."""
        parts = [g for g in self.groups if g.partition_params]
        for g in parts:
            g.gather()
        try:
            yield
        finally:
            for g in parts:
                if write_back:
                    g.store_shard_from_gathered()
                g.release()

    # ------------------------------------------------------------------ reference-engine surface
    def train(self, mode=True):
        super().train(mode)
        return self

    def forward(self, *inputs, **kwargs):
        # sequence-length curriculum: while training, the current difficulty is handed to the model, which
        # truncates the batch to it (models/utils.py SequentialWrapper.forward) and records it in the arguments
        # so that the loss side truncates labels and mask the same way
        sched = getattr(self, "curriculum_scheduler", None)
        if sched is not None and self.module.training and "curriculum_seqlen" not in kwargs:
            kwargs["curriculum_seqlen"] = sched.update_difficulty(self.global_steps + 1)
        if self.flops_profiler is not None and self.module.training:
            self.flops_profiler.before_forward(self.global_steps + 1)
        with self._span("forward"):
            return self.module(*inputs, **kwargs)

    def _span(self, phase):
        return self.breakdown.span(phase) if self.breakdown is not None else contextlib.nullcontext()

    def is_gradient_accumulation_boundary(self):
        return (self.micro_steps + 1) % self.gradient_accumulation_steps == 0

    @property
    def cur_scale(self):
        return self.loss_scaler.cur_scale

    def get_global_grad_norm(self):
        return None if self._last_grad_norm is None else float(self._last_grad_norm)

    def backward(self, loss, retain_graph=False):
        """Scale by 1/GAS (and the fp16 loss scale) and back-propagate."""
        scaled = loss / self.gradient_accumulation_steps
        if self.fp16_enabled:
            scaled = scaled * self.loss_scaler.cur_scale
        with self._span("backward"):
            scaled.backward(retain_graph=retain_graph)
            self._z3_finish()
            self._ov_finish()
        return loss

    def _sync_sequence_parallel_grads(self):
        """Norm parameters see only their sequence shard under sequence parallelism: sum their
        gradients over the tensor-parallel group with ONE flat all-reduce."""
        if mpu.get_model_parallel_world_size() == 1:
            return
        ps = [p for g in self.groups for p in g.params if getattr(p, "sequence_parallel_grad_sync", False)]
        if not ps:
            return
        flat = torch.cat([p.main_grad.reshape(-1) for p in ps])
        dist.all_reduce(flat, group=mpu.get_model_parallel_group())
        off = 0
        for p in ps:
            n = p.numel()
            p.main_grad.copy_(flat[off:off + n].view_as(p.main_grad))
            off += n

    def step(self):
        """Optimizer step at the accumulation boundary, otherwise just count the micro-step."""
        boundary = self.is_gradient_accumulation_boundary()
        self.micro_steps += 1
        self.global_samples += self.neox_args.train_micro_batch_size_per_gpu * mpu.get_data_parallel_world_size()
        if not boundary:
            return
        self._take_model_step()

    def _take_model_step(self):
        for g in self.groups:
            g.fold_autograd_grads()
        self._sync_sequence_parallel_grads()
        if self.store_gradients:
            self.stored_gradients = [p.main_grad.detach().clone() for g in self.groups for p in g.params]
        # 1-bit Adam past its warm-up averages compressed momenta itself: the gradients stay local
        local_grads = bool(self.optimizer is not None and self.optimizer.generic is not None
                           and getattr(self.optimizer.generic, "wants_local_gradients", lambda: False)())
        with self._span("grad_reduce"):
            for g in self.groups:
                if not local_grads:
                    g.reduce_gradients()
        # global gradient norm: every element is owned (counted) by exactly one rank of the world
        self._acc.zero_()
        tp_rank0 = mpu.get_model_parallel_rank() == 0
        for g in self.groups:
            if not g.sharded and g.dp_size > 1 and g.dp_rank != 0:
                continue       # unsharded group (ZeRO stage 0): every data-parallel rank holds the same reduced
                               # gradient, so only the first one counts it
            gs = g.grad_shard()
            for (lo, hi, _wd, rep, skip, _lrm) in g.segments:
                if skip or (rep and not tp_rank0):
                    continue   # counted by another owner (tensor-parallel replica / tied pipeline copy)
                optim_ops.sumsq_(gs[lo:hi], self._acc)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self._acc[0:1])
            dist.all_reduce(self._acc[1:2], op=dist.ReduceOp.MAX)
        dp_avg = 1.0 / max(g.dp_size for g in self.groups) if self.groups else 1.0
        dp_avg *= self._predivide                      # undo what reduce_gradients divided by beforehand
        if local_grads:
            dp_avg = 1.0                               # nothing was summed
        inv_scale = dp_avg / (self.loss_scaler.cur_scale if self.fp16_enabled else 1.0)
        optim_ops.clip_coef_(self._acc, self.gradient_clipping, inv_scale, self._scale, self._skip)
        self._last_grad_norm = self._scale[1]
        overflow = False
        if self.fp16_enabled:
            overflow = bool(self._skip.item() != 0)     # fp16 only: the scaler needs the answer on the host
            self.loss_scaler.update_scale(overflow)
        if self.optimizer is not None:
            self.optimizer.overflow = overflow
            self.optimizer.cur_scale = self.loss_scaler.cur_scale
            with self._span("optimizer"):
                self.optimizer.step(self._scale, self._skip)
        with self._span("param_gather"):
            for g in self.groups:
                g.gather_params()
                g.zero_grad()
        if self.groups and self.groups[0].device.type == "cuda":
            from ..comm import symm
            symm.pool_reset_all()           # no gathered activation outlives the step: every gather-pool slot is free
        for m in self._fp8_modules():
            m.fp8_meta.roll()               # delayed scaling: this step's amax feeds the next steps' scales
        if getattr(self.neox_args, "te_fp8_recipe", "delayed") == "mxfp8":
            from ..ops import fp8
            fp8.mxfp8_new_step()            # block scaling: the weights changed, their quantised copies are stale
        if overflow:
            self.skipped_steps += 1
        elif self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.global_steps += 1
        if self.flops_profiler is not None:
            self.flops_profiler.after_step(self.global_steps)
        if self.breakdown is not None:
            self.breakdown.end_step(self)

    def _fp8_modules(self):
        return [m for m in self.module.modules() if getattr(m, "fp8_meta", None) is not None]

    def zero_grad(self):
        for g in self.groups:
            g.zero_grad()

    def set_batch_fn(self, fn):
        self.batch_fn = fn
        if hasattr(self.module, "set_batch_fn"):
            self.module.set_batch_fn(fn)

    def set_has_attention_mask(self, value):
        self.has_attention_mask = value

    @property
    def total_params(self):
        return sum(g.numel() for g in self.groups)

    # checkpoint IO is implemented in ckpt/ and bound here
    def save_checkpoint(self, save_dir, tag=None, client_state=None):
        from ..ckpt.io import save_engine_checkpoint
        return save_engine_checkpoint(self, save_dir, tag, client_state or {})

    def load_checkpoint(self, load_dir, tag=None, load_optimizer_states=True, load_lr_scheduler_states=True,
                        load_module_only=False, load_module_strict=True):
        from ..ckpt.io import load_engine_checkpoint
        return load_engine_checkpoint(self, load_dir, tag, load_optimizer_states, load_lr_scheduler_states,
                                      load_module_only, load_module_strict)


def initialize(model, neox_args, param_groups=None, optimizer_cfg=None, lr_scheduler=None, generic_optimizer=None):
    """Counterpart of ``deepspeed.initialize``: returns ``(engine, optimizer, None, lr_scheduler)``.
    A pipeline-parallel model gets the pipeline engine."""
    if param_groups is None:
        from ..models.utils import get_params_for_weight_decay_optimization
        param_groups = get_params_for_weight_decay_optimization(model, neox_args)
    if neox_args.is_pipe_parallel:
        from .pipeline import PipelineEngine
        engine = PipelineEngine(model, neox_args, param_groups, optimizer_cfg, lr_scheduler, generic_optimizer)
    else:
        engine = Engine(model, neox_args, param_groups, optimizer_cfg, lr_scheduler, generic_optimizer)
    if lr_scheduler is not None and engine.optimizer is not None:
        lr_scheduler.optimizer = engine.optimizer
        lr_scheduler.step(lr_scheduler.num_iters)
    return engine, engine.optimizer, None, lr_scheduler
