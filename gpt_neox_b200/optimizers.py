"""In-tree optimizers other than AdamW: SM3, MADGRAD with decoupled weight decay, Lion
(megatron/optimizers.py:20-497).  Dense gradients only: the engine hands every optimizer fp32 views of
its flat master-weight shard, so the sparse-gradient branches of the reference have no caller here.

All three share one skeleton (`_PerTensor`): per-tensor state created on first use, one `_apply` call
per parameter under ``torch.no_grad``.
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer


class _PerTensor(Optimizer):
    def _new_state(self, p, group):           # -> dict
        raise NotImplementedError

    def _apply(self, p, g, st, group):
        raise NotImplementedError

    def _before_step(self):
        pass

    def _after_step(self):
        pass

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if callable(closure):
            with torch.enable_grad():
                loss = closure()
        self._before_step()
        for group in self.param_groups:
            for p in group["params"]:
                if p is None or p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError(f"{type(self).__name__}: sparse gradients are not supported")
                st = self.state[p]
                if not st:
                    st.update(self._new_state(p, group))
                self._apply(p, p.grad, st, group)
        self._after_step()
        return loss


class SM3(_PerTensor):
    """Memory-efficient adaptive optimisation (arXiv:1901.11150): a rank-n tensor keeps n cover
    accumulators of shapes (d_0,1,..), (1,d_1,..), ...; the second-moment estimate of an entry is the
    minimum over its covers, and each cover is refreshed with the maximum of the estimates it spans."""

    def __init__(self, params, lr=0.1, momentum=0.0, beta=0.0, eps=1e-30):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 <= momentum < 1.0:
            raise ValueError(f"Invalid momentum: {momentum}")
        if not 0.0 <= beta < 1.0:
            raise ValueError(f"Invalid beta: {beta}")
        if eps < 0.0:
            raise ValueError(f"Invalid eps: {eps}")
        super().__init__(params, {"lr": lr, "momentum": momentum, "beta": beta, "eps": eps})

    def _new_state(self, p, group):
        shape = p.shape
        covers = []
        if p.dim() == 0:
            covers.append(torch.zeros_like(p))
        else:
            for axis, n in enumerate(shape):
                s = [1] * p.dim()
                s[axis] = n
                covers.append(torch.zeros(s, device=p.device, dtype=p.dtype))
        return {"step": 0, "covers": covers, "momentum_buffer": None}

    def _apply(self, p, g, st, group):
        beta, mom, eps = group["beta"], group["momentum"], group["eps"]
        covers = st["covers"]
        nu = covers[0]
        for c in covers[1:]:
            nu = torch.minimum(nu, c)                       # broadcasts to the full shape
        nu = nu * beta + (1.0 - beta) * g * g if beta > 0.0 else nu + g * g
        for axis, c in enumerate(covers):
            m = nu
            for d in range(nu.dim()):
                if d != axis:
                    m = m.amax(dim=d, keepdim=True)
            if beta > 0.0:
                torch.maximum(c, m, out=c)
            else:
                c.copy_(m)
        upd = g * torch.rsqrt(nu + eps)
        if mom > 0.0:
            buf = st["momentum_buffer"]
            upd = upd * (1.0 - mom) + (buf * mom if buf is not None else 0.0)
            st["momentum_buffer"] = upd.clone()
        p.sub_(upd, alpha=group["lr"])
        st["step"] += 1


class madgrad_wd(_PerTensor):
    """MADGRAD (arXiv:2101.11075) with AdamW-style decoupled weight decay: dual averaging of the
    gradients with a cube-root second-moment denominator, momentum as interpolation towards the
    dual-averaged iterate."""

    def __init__(self, params, lr=1e-2, momentum=0.9, weight_decay=0, eps=1e-6):
        if not 0 <= momentum < 1:
            raise ValueError(f"Momentum {momentum} must be in the range [0,1]")
        if lr <= 0:
            raise ValueError(f"Learning rate {lr} must be positive")
        if weight_decay < 0:
            raise ValueError(f"Weight decay {weight_decay} must be non-negative")
        if eps < 0:
            raise ValueError("Eps must be non-negative")
        super().__init__(params, dict(lr=lr, eps=eps, momentum=momentum, weight_decay=weight_decay))
        self._k = 0

    supports_memory_efficient_fp16 = False
    supports_flat_params = True

    def _new_state(self, p, group):
        st = {"grad_sum_sq": torch.zeros_like(p), "s": torch.zeros_like(p)}
        if group["momentum"] != 0:
            st["x0"] = p.detach().clone()
        return st

    def _apply(self, p, g, st, group):
        eps, mom, decay = group["eps"], group["momentum"], group["weight_decay"]
        lr = group["lr"] + eps
        lamb = lr * math.sqrt(self._k + 1)
        nu, s = st["grad_sum_sq"], st["s"]
        if decay:
            p.mul_(1 - lr * decay)
        if mom == 0:
            x0 = p + s / (nu.pow(1 / 3) + eps)              # recover the anchor from the current iterate
        else:
            x0 = st["x0"]
        nu.addcmul_(g, g, value=lamb)
        s.add_(g, alpha=lamb)
        z = x0 - s / (nu.pow(1 / 3) + eps)
        if mom == 0:
            p.copy_(z)
        else:
            p.mul_(mom).add_(z, alpha=1 - mom)

    def _after_step(self):
        self._k += 1

    def state_dict(self):
        sd = super().state_dict()
        sd["k"] = self._k
        return sd

    def load_state_dict(self, sd):
        self._k = sd.pop("k", 0) if isinstance(sd, dict) else 0
        super().load_state_dict(sd)


class Lion(_PerTensor):
    """Lion (arXiv:2302.06675): sign of an interpolated momentum, decoupled weight decay, a single
    moment buffer."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        if lr <= 0:
            raise ValueError(f"Learning rate {lr} must be positive")
        if weight_decay < 0:
            raise ValueError(f"Weight decay {weight_decay} must be non-negative")
        if not (0 <= betas[0] <= 1 and 0 <= betas[1] <= 1):
            raise ValueError(f"Betas {betas} must be in range [0, 1)")
        super().__init__(params, dict(lr=lr, betas=tuple(betas), weight_decay=weight_decay))

    def _new_state(self, p, group):
        return {"exp_avg": torch.zeros_like(p)}

    def _apply(self, p, g, st, group):
        b1, b2 = group["betas"]
        m = st["exp_avg"]
        p.mul_(1 - group["lr"] * group["weight_decay"])
        p.add_(torch.sign(m * b1 + g * (1 - b1)), alpha=-group["lr"])
        m.mul_(b2).add_(g, alpha=1 - b2)


# ------------------------------------------------------------------------------------------------------------------
# 1-bit Adam
# ------------------------------------------------------------------------------------------------------------------
def _pack_signs(x: torch.Tensor) -> torch.Tensor:
    """One bit per element (1 = non-negative), eight elements per byte; ``x.numel() % 8 == 0``."""
    bits = (x >= 0).view(-1, 8).to(torch.uint8)
    w = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.uint8, device=x.device)
    return (bits * w).sum(dim=1, dtype=torch.uint8)


def _unpack_signs(b: torch.Tensor) -> torch.Tensor:
    """Bytes -> a float tensor of +1 / -1, eight per byte."""
    sh = torch.arange(8, device=b.device, dtype=torch.uint8)
    bits = (b.view(-1, 1) >> sh) & 1
    return bits.to(torch.float32).mul_(2.0).sub_(1.0).view(-1)


class CompressedAllreduce:
    """Error-compensated 1-bit average of a flat fp32 vector over a process group: the two-stage scheme of 1-bit
    Adam (each rank sends one bit per element plus one scale; rank r serves chunk r: it averages what it received,
    compresses the average again with its own error feedback, and the served chunks are gathered back).  Both
    quantisation errors are kept and added to the next call's input, so nothing is lost over time.  Works on NCCL
    and gloo; traffic per rank is n / 4 bytes per call instead of 8 n for an fp32 all-reduce."""

    def __init__(self, numel: int, group, device):
        import torch.distributed as dist
        self.group = group
        self.ws = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.ws > 1 else 0
        unit = 8 * self.ws
        self.numel = numel
        self.padded = (numel + unit - 1) // unit * unit
        self.chunk = self.padded // self.ws
        self.worker_error = torch.zeros(self.padded, dtype=torch.float32, device=device)
        self.server_error = torch.zeros(self.chunk, dtype=torch.float32, device=device)

    @staticmethod
    def _compress(x, error):
        """x += error; returns (packed signs, scale) and leaves the new quantisation error in ``error``."""
        x.add_(error)
        scale = x.norm() / math.sqrt(x.numel())
        signs = torch.where(x >= 0, 1.0, -1.0)
        torch.sub(x, scale * signs, out=error)
        return _pack_signs(x), scale

    @torch.no_grad()
    def __call__(self, vec: torch.Tensor) -> torch.Tensor:
        """In place: ``vec`` (fp32, ``numel`` elements) becomes the compressed average over the group."""
        import torch.distributed as dist
        buf = torch.zeros(self.padded, dtype=torch.float32, device=vec.device)
        buf[: self.numel].copy_(vec)
        packed, scale = self._compress(buf, self.worker_error)
        if self.ws == 1:
            vec.copy_((_unpack_signs(packed) * scale)[: self.numel])
            return vec
        # stage 1: chunk r of every rank's signs goes to rank r; all scales go everywhere
        recv = torch.empty_like(packed)
        dist.all_to_all_single(recv, packed, group=self.group)
        scales = [torch.empty_like(scale.reshape(1)) for _ in range(self.ws)]
        dist.all_gather(scales, scale.reshape(1), group=self.group)
        per = self.chunk // 8
        served = torch.zeros(self.chunk, dtype=torch.float32, device=vec.device)
        for r in range(self.ws):
            served.add_(_unpack_signs(recv[r * per:(r + 1) * per]) * scales[r])
        served.div_(self.ws)
        # stage 2: compress the served chunk again (server error feedback) and gather all chunks
        s_packed, s_scale = self._compress(served, self.server_error)
        all_packed = [torch.empty_like(s_packed) for _ in range(self.ws)]
        dist.all_gather(all_packed, s_packed, group=self.group)
        s_scales = [torch.empty_like(s_scale.reshape(1)) for _ in range(self.ws)]
        dist.all_gather(s_scales, s_scale.reshape(1), group=self.group)
        out = torch.cat([_unpack_signs(all_packed[r]) * s_scales[r] for r in range(self.ws)])
        vec.copy_(out[: self.numel])
        return vec


class OnebitAdam(Optimizer):
    """1-bit Adam (the optimizer the reference obtains from DeepSpeed for ``"type": "OneBitAdam"``,
    megatron/training.py:1014-1017): Adam for ``freeze_step`` warm-up steps on fully reduced gradients; afterwards
    the second moment is frozen, every rank folds its LOCAL gradient into the momentum and the momenta are averaged
    by the error-compensated 1-bit all-reduce above (32 x less traffic than the gradient all-reduce it replaces).
    Update rule as in DeepSpeed's implementation: no bias correction, weight decay added to the update.

    The engine asks ``wants_local_gradients()`` before each step and leaves the data-parallel gradient reduction
    out when it returns True.  Needs unpartitioned optimizer state (ZeRO stage 0), like the original."""

    def __init__(self, params, lr=1e-3, freeze_step=100000, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 comm_group=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.freeze_step = int(freeze_step)
        self.comm_group = comm_group
        self.steps = 0
        self.compression_steps = 0
        self._comm = None

    def wants_local_gradients(self) -> bool:
        return self.steps >= self.freeze_step

    def _params(self):
        return [(g, p) for g in self.param_groups for p in g["params"] if p.grad is not None]

    @torch.no_grad()
    def step(self, closure=None):
        compress = self.wants_local_gradients()
        self.steps += 1
        items = self._params()
        for g, p in items:
            st = self.state[p]
            if not st:
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            b1, b2 = g["betas"]
            st["exp_avg"].mul_(b1).add_(p.grad.float(), alpha=1 - b1)
            if not compress:
                st["exp_avg_sq"].mul_(b2).addcmul_(p.grad.float(), p.grad.float(), value=1 - b2)
        if compress and items:
            # one compressed all-reduce for the momenta of all parameters
            flat = torch.cat([self.state[p]["exp_avg"].reshape(-1) for _, p in items])
            if self._comm is None or self._comm.numel != flat.numel():
                group = self.comm_group
                if group is None:
                    from . import parallel as mpu
                    group = mpu.get_data_parallel_group()
                self._comm = CompressedAllreduce(flat.numel(), group, flat.device)
                pend = getattr(self, "_pending_errors", None)        # error feedback of a resumed run
                if pend is not None and pend[0] is not None and pend[0].numel() == self._comm.worker_error.numel():
                    self._comm.worker_error.copy_(pend[0])
                    self._comm.server_error.copy_(pend[1])
                self._pending_errors = None
            self._comm(flat)
            off = 0
            for _, p in items:
                n = p.numel()
                self.state[p]["exp_avg"].copy_(flat[off:off + n].view_as(p))
                off += n
            self.compression_steps += 1
        for g, p in items:
            st = self.state[p]
            update = st["exp_avg"] / (st["exp_avg_sq"].sqrt() + g["eps"])
            if g["weight_decay"] > 0:
                update.add_(p.float(), alpha=g["weight_decay"])
            p.add_(update.to(p.dtype), alpha=-g["lr"])

    def state_dict(self):
        sd = super().state_dict()
        sd["onebit"] = {"steps": self.steps, "compression_steps": self.compression_steps,
                        "worker_error": None if self._comm is None else self._comm.worker_error.cpu(),
                        "server_error": None if self._comm is None else self._comm.server_error.cpu()}
        return sd

    def load_state_dict(self, sd):
        extra = sd.pop("onebit", None) if isinstance(sd, dict) else None
        super().load_state_dict(sd)
        if extra:
            self.steps, self.compression_steps = extra["steps"], extra["compression_steps"]
            self._pending_errors = (extra["worker_error"], extra["server_error"])
