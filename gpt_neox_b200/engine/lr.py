"""Learning-rate schedule: linear warm-up, then constant / linear / cosine / exponential decay to
``min_lr`` (megatron/learning_rates.py:25-148), with the checkpoint override rules
(``use_checkpoint_lr_scheduler`` / ``override_lr_scheduler``) and muP per-group width scaling."""
from __future__ import annotations

import math


class AnnealingLR:
    def __init__(self, optimizer, start_lr, warmup_iter, total_iters, decay_style, last_iter, min_lr=0.0,
                 use_checkpoint_lr_scheduler=True, override_lr_scheduler=False, use_mup=False):
        self.optimizer = optimizer
        self.start_lr, self.min_lr = start_lr, min_lr
        self.warmup_iter = warmup_iter
        self.num_iters = last_iter
        self.end_iter = total_iters
        assert self.end_iter > 0
        self.decay_style = decay_style
        self.override_lr_scheduler = override_lr_scheduler
        self.use_checkpoint_lr_scheduler = use_checkpoint_lr_scheduler
        self.use_mup = use_mup
        if self.override_lr_scheduler:
            assert not self.use_checkpoint_lr_scheduler, "both override and use-checkpoint are set."
        self.step(self.num_iters)

    def get_lr(self):
        n = self.num_iters
        if self.warmup_iter > 0 and n <= self.warmup_iter:
            return float(self.start_lr) * max(1, n) / self.warmup_iter
        n = n - self.warmup_iter
        span = self.end_iter - self.warmup_iter
        if self.decay_style == "linear":
            lr = self.start_lr * (span - n) / span
        elif self.decay_style == "cosine":
            lr = self.min_lr + (self.start_lr - self.min_lr) / 2.0 * (math.cos(math.pi * n / span) + 1)
        elif self.decay_style == "exponential":
            lr = self.start_lr * math.exp(-0.693 * n / span)
        else:
            lr = self.start_lr
        return max(lr, self.min_lr)

    def step(self, step_num=None):
        if step_num is None:
            step_num = self.num_iters + 1
        self.num_iters = step_num
        new_lr = self.get_lr()
        for group in self.optimizer.param_groups:
            if self.use_mup and "width_mult" in group:
                group["lr"] = new_lr / group["width_mult"]
            else:
                group["lr"] = new_lr

    def state_dict(self):
        return {"start_lr": self.start_lr, "warmup_iter": self.warmup_iter, "num_iters": self.num_iters,
                "decay_style": self.decay_style, "end_iter": self.end_iter, "min_lr": self.min_lr}

    def _check_and_set(self, cls_value, sd_value, name):
        if self.override_lr_scheduler:
            return cls_value
        if not self.use_checkpoint_lr_scheduler:
            assert cls_value == sd_value, \
                f"AnnealingLR: class input value and checkpoint values for {name} do not match"
        return sd_value

    def load_state_dict(self, sd):
        self.start_lr = self._check_and_set(self.start_lr, sd["start_lr"], "learning rate")
        self.min_lr = self._check_and_set(self.min_lr, sd["min_lr"], "minimum learning rate")
        self.warmup_iter = self._check_and_set(self.warmup_iter, sd["warmup_iter"], "warmup iterations")
        self.end_iter = self._check_and_set(self.end_iter, sd["end_iter"], "total number of iterations")
        self.decay_style = self._check_and_set(self.decay_style, sd["decay_style"], "decay style")
        self.num_iters = sd["num_iters"]
        self.step(self.num_iters)
