"""Gradient noise scale B_simple = tr(Sigma) / |G|^2 (arXiv:1812.06162), estimated from the squared gradient
norms at two batch sizes: one optimizer step (B_small) and the mean gradient over ``n_batches`` consecutive
steps (B_big), with exponential moving averages of both estimators
(megatron/gradient_noise_scale/gradient_noise_scale.py:26-210).

The engine keeps gradients in one flat fp32 buffer per group, so "the gradient" is that buffer: the
running sum costs one ``add_`` per group per step and no per-parameter flattening.
"""
from __future__ import annotations

import torch


def ema(avg, beta, yi, i):
    """Bias-corrected exponential moving average: returns (new raw average, corrected value)."""
    avg = 0.0 if avg is None else avg
    avg = beta * avg + (1 - beta) * yi
    return avg, avg / (1 - beta ** (i + 1))


class GradientNoiseScale:
    def __init__(self, model, batch_size_small, n_batches=10, beta=0.99, cpu_offload=False, neox_args=None, mpu=None):
        self.batch_size_small = batch_size_small
        self.batch_size_large = batch_size_small * n_batches
        self.n_batches, self.beta = n_batches, beta
        self.model = model
        self.buffer = None
        self.ema_scale = self.ema_noise = self.noise_scale = None
        self.n_updates = 0
        self.cpu_offload = cpu_offload
        self.model.store_gradients = True
        self.model.store_gradients_cpu = cpu_offload
        self.neox_args, self.mpu = neox_args, mpu

    def flatten_grads(self):
        grads = getattr(self.model, "stored_gradients", None)
        if not grads:
            return None
        flat = torch.cat([g.reshape(-1).float() for g in grads if g is not None])
        if not bool(torch.isfinite(flat).all()):
            return None
        return flat.cpu() if self.cpu_offload else flat

    def _pipe(self):
        return bool(self.neox_args is not None and self.neox_args.is_pipe_parallel and
                    torch.distributed.is_initialized() and self.mpu.get_pipe_parallel_world_size() > 1)

    def _sync_overflow(self, flag: bool) -> bool:
        if not self._pipe():
            return bool(flag)
        t = torch.tensor([int(flag)], dtype=torch.int32, device=self._dev())
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=self.mpu.get_pipe_parallel_group())
        return bool(t.item())

    def _dev(self):
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")

    def _sq_norm(self, x):
        v = torch.sum(x.float() * x.float()).to(self._dev())
        if self._pipe():
            torch.distributed.all_reduce(v, group=self.mpu.get_pipe_parallel_group())
            v = v / self.mpu.get_pipe_parallel_world_size()
        return v

    def _update(self):
        grad = self.flatten_grads()
        if self._sync_overflow(grad is None):
            return
        self.buffer = grad.clone() if self.buffer is None else self.buffer.add_(grad)
        if self.n_updates % self.n_batches == self.n_batches - 1:
            big = self.buffer / self.n_batches
            self.buffer = None
            g_big, g_small = self._sq_norm(big), self._sq_norm(grad)
            bad = not bool(torch.isfinite(g_big)) or not bool(torch.isfinite(g_small))
            if self._sync_overflow(bad):
                return
            bs, bl = self.batch_size_small, self.batch_size_large
            noise = (bl * g_big - bs * g_small) / (bl - bs)                 # estimates |G|^2
            scale = (g_small - g_big) / (1.0 / bs - 1.0 / bl)               # estimates tr(Sigma)
            self.ema_noise, noise = ema(self.ema_noise, self.beta, noise, self.n_updates)
            self.ema_scale, scale = ema(self.ema_scale, self.beta, scale, self.n_updates)
            self.noise_scale = float(scale) / float(noise)
        self.n_updates += 1

    def update(self):
        if self._pipe() or not torch.distributed.is_initialized():
            self._update()
        else:
            if torch.distributed.get_rank() == 0:
                self._update()
            torch.distributed.barrier()
