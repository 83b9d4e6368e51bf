"""fp16 loss scaling: static, or dynamic with the engine keys the reference passes through
(``loss_scale``, ``initial_scale_power``, ``loss_scale_window``, ``hysteresis``, ``min_loss_scale`` —
configs/pythia/6-9B.yml): halve on overflow after ``hysteresis`` consecutive overflows, double after
``loss_scale_window`` clean steps."""
from __future__ import annotations


class LossScaler:
    def __init__(self, scale=1.0):
        self.cur_scale = float(scale)
        self.dynamic = False

    def update_scale(self, overflow: bool):
        pass

    def state_dict(self):
        return {"cur_scale": self.cur_scale}

    def load_state_dict(self, sd):
        self.cur_scale = sd.get("cur_scale", self.cur_scale)


class DynamicLossScaler(LossScaler):
    def __init__(self, init_scale=2 ** 32, scale_factor=2.0, scale_window=1000, min_scale=1.0, hysteresis=2,
                 consecutive_hysteresis=False):
        super().__init__(init_scale)
        self.dynamic = True
        self.cur_iter = 0
        self.last_overflow_iter = -1
        self.scale_factor, self.scale_window, self.min_scale = scale_factor, int(scale_window), min_scale
        self.delayed_shift = hysteresis
        self.cur_hysteresis = hysteresis
        self.consecutive_hysteresis = consecutive_hysteresis

    def update_scale(self, overflow: bool):
        if overflow:
            if self.delayed_shift == 1 or self.cur_hysteresis == 1:
                self.cur_scale = max(self.cur_scale / self.scale_factor, self.min_scale)
            else:
                self.cur_hysteresis -= 1
            self.last_overflow_iter = self.cur_iter
        else:
            if self.consecutive_hysteresis:
                self.cur_hysteresis = self.delayed_shift
            if (self.cur_iter - self.last_overflow_iter) % self.scale_window == 0:
                if not self.consecutive_hysteresis:
                    self.cur_hysteresis = self.delayed_shift
                self.cur_scale *= self.scale_factor
        self.cur_iter += 1

    def state_dict(self):
        return {"cur_scale": self.cur_scale, "cur_iter": self.cur_iter, "last_overflow_iter": self.last_overflow_iter,
                "cur_hysteresis": self.cur_hysteresis}

    def load_state_dict(self, sd):
        self.cur_scale = sd.get("cur_scale", self.cur_scale)
        self.cur_iter = sd.get("cur_iter", 0)
        self.last_overflow_iter = sd.get("last_overflow_iter", -1)
        self.cur_hysteresis = sd.get("cur_hysteresis", self.delayed_shift)


def build_loss_scaler(fp16_cfg: dict | None):
    cfg = fp16_cfg or {}
    static = cfg.get("loss_scale", 0)
    if static and static > 0:
        return LossScaler(static)
    return DynamicLossScaler(init_scale=2 ** cfg.get("initial_scale_power", 16),
                             scale_window=cfg.get("loss_scale_window", 1000),
                             min_scale=cfg.get("min_loss_scale", 1),
                             hysteresis=cfg.get("hysteresis", 2),
                             consecutive_hysteresis=cfg.get("consecutive_hysteresis", False))
