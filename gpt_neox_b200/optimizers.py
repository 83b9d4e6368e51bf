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
