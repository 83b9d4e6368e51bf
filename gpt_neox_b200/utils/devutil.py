"""Developer aid: time every call of one method and keep the distribution.

Counterpart of megatron/devutil.py:4-51 (``Metric`` + ``monitor_method_cuda_wall_times``).  The timing
uses CUDA events on the current stream when the process has a GPU and the host clock otherwise;
``restore()`` puts the original method back.

    metric = Metric("layernorm forward")
    undo = monitor_method_wall_times(metric, LayerNorm, "forward")
    ...
    metric.report(); undo()
"""
from __future__ import annotations

import time

import torch


class Metric:
    def __init__(self, label: str):
        self.label = label
        self.measurements = []

    def collect(self, measurement: float):
        self.measurements.append(float(measurement))

    def get_measurements(self):
        return list(self.measurements)

    def deciles(self):
        if not self.measurements:
            return torch.empty(0)
        return torch.quantile(torch.tensor(self.measurements, dtype=torch.float64), torch.arange(10, dtype=torch.float64) / 10.0)

    def report(self, out=print):
        out(f"{self.label}: n={len(self.measurements)} deciles (ms)="
            f"{[round(float(v), 4) for v in self.deciles()]}")


def monitor_method_wall_times(metric: Metric, obj, methodname: str, report_every: int = 0):
    """Wrap ``obj.methodname`` so that each call's duration in milliseconds is collected into ``metric``
    (and reported every ``report_every`` calls when > 0).  Returns the function that undoes the wrapping."""
    original = getattr(obj, methodname)
    use_cuda = torch.cuda.is_available()

    def timed(*args, **kwargs):
        if use_cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        else:
            t0 = time.perf_counter()
        try:
            return original(*args, **kwargs)
        finally:
            if use_cuda:
                b.record()
                b.synchronize()
                metric.collect(a.elapsed_time(b))
            else:
                metric.collect((time.perf_counter() - t0) * 1e3)
            if report_every and len(metric.measurements) % report_every == 0:
                metric.report()

    setattr(obj, methodname, timed)

    def restore():
        setattr(obj, methodname, original)
    return restore


monitor_method_cuda_wall_times = monitor_method_wall_times
