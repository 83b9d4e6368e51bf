"""Engine-side observability switches: ``wall_clock_breakdown``, ``flops_profiler``, ``comms_logger``, ``dump_state``.

The reference only declares these keys (megatron/neox_arguments/deepspeed_args.py:146-173,238) and lets the
DeepSpeed engine act on them; its logging reads the result back as ``model.timer_values``
(megatron/logging.py:299-319).  Here the engine owns them:

* `StepBreakdown`: time per phase of a step (forward, backward, gradient reduction, optimizer, parameter
  gather, pipeline transfers), taken with CUDA events on the launching stream (host clock on CPU) and
  resolved only when a line is printed, so that no step waits for the host;
* `FlopsProfiler`: at one chosen step, forward hooks time every module and count its matrix-multiply
  FLOPs from the shapes that pass through; the report is a per-depth table (parameters, FLOPs, latency);
* `CommsLogger`: wraps the ``torch.distributed`` collectives (and this framework's own NVLink collectives,
  which report through `observe`) and tabulates count, message size, latency, algorithm and bus bandwidth.
"""
from __future__ import annotations

import contextlib
import sys
import time
from collections import OrderedDict, defaultdict

import torch
import torch.distributed as dist


def _rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


# ---------------------------------------------------------------------------------------- step breakdown
class StepBreakdown:
    PHASES = ("forward", "backward", "grad_reduce", "optimizer", "param_gather", "pipe_comm")

    def __init__(self, steps_per_print=10, device=None, out=None):
        self.steps_per_print = max(1, int(steps_per_print or 10))
        self.cuda = device is not None and torch.device(device).type == "cuda"
        self.pending = []                  # (phase, start, end): events on CUDA, floats on CPU
        self.steps = 0
        self.out = out
        self.last = None

    @contextlib.contextmanager
    def span(self, phase):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self.pending.append((phase, a, b))
        else:
            t = time.perf_counter()
            try:
                yield
            finally:
                self.pending.append((phase, t, time.perf_counter()))

    def end_step(self, engine=None):
        """Count a finished step; every ``steps_per_print`` steps resolve the spans, publish the means as
        ``engine.timer_values`` (milliseconds per step) and print them on rank 0."""
        self.steps += 1
        if self.steps % self.steps_per_print:
            return None
        total = defaultdict(float)
        if self.cuda and self.pending:
            self.pending[-1][2].synchronize()
        for phase, a, b in self.pending:
            total[phase] += a.elapsed_time(b) if self.cuda else (b - a) * 1e3
        self.pending = []
        vals = OrderedDict((p, total[p] / self.steps_per_print) for p in self.PHASES if p in total)
        self.last = vals
        if engine is not None:
            engine.timer_values = dict(vals)
        if _rank() == 0:
            line = "time (ms) per step | " + " | ".join(f"{k}: {v:.2f}" for k, v in vals.items())
            print(line, file=self.out or sys.stdout, flush=True)
        return vals


# ---------------------------------------------------------------------------------------- flops profiler
def _numel(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _first_tensor(x):
    if torch.is_tensor(x):
        return x
    if isinstance(x, (tuple, list)):
        for y in x:
            t = _first_tensor(y)
            if t is not None:
                return t
    return None


def module_forward_flops(mod, inputs, output) -> float:
    """Matrix-multiply FLOPs of one forward call of ``mod`` itself (children are counted at their own hook)."""
    x = _first_tensor(inputs)
    name = type(mod).__name__
    w = getattr(mod, "weight", None)
    if x is not None and torch.is_tensor(w) and w.dim() == 2 and x.is_floating_point() and "Embedding" not in name:
        return 2.0 * (x.numel() / max(1, x.shape[-1])) * w.numel()
    if "SelfAttention" in name and x is not None and x.dim() == 3:
        s, b = x.shape[0], x.shape[1]
        hp = getattr(mod, "hidden_size_per_partition", None) or x.shape[-1]
        sp = getattr(mod, "sequence_parallel", False)
        if sp:
            s = s * getattr(mod, "world_size", 1)
        return 4.0 * b * s * s * hp                     # Q K^T and P V, uncausal count
    if x is not None and any(torch.is_tensor(p) and p.dim() == 3 for p in mod._parameters.values()):
        tokens = x.numel() / max(1, x.shape[-1])        # grouped expert weights [experts, in, out]
        k = getattr(mod, "top_k", None) or getattr(mod, "moe_top_k", 1) or 1
        per = sum(p.numel() / p.shape[0] for p in mod._parameters.values() if torch.is_tensor(p) and p.dim() == 3)
        return 2.0 * tokens * k * per
    return 0.0


class FlopsProfiler:
    def __init__(self, model, profile_step=1, module_depth=-1, top_modules=1, detailed=True, output_file=None):
        self.model = model
        self.profile_step = int(profile_step)
        self.module_depth = int(module_depth)
        self.top_modules = int(top_modules)
        self.detailed = bool(detailed)
        self.output_file = output_file
        self.handles, self.stats, self.started = [], {}, False

    @classmethod
    def from_args(cls, model, neox_args):
        cfg = getattr(neox_args, "flops_profiler", None) or {}
        if not cfg.get("enabled"):
            return None
        keys = ("profile_step", "module_depth", "top_modules", "detailed", "output_file")
        return cls(model, **{k: cfg[k] for k in keys if k in cfg})

    def _sync(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def start(self):
        self.stats = {}
        for name, mod in self.model.named_modules():
            st = self.stats[name] = dict(flops=0.0, ms=0.0, calls=0, cls=type(mod).__name__,
                                         params=sum(p.numel() for p in mod.parameters(recurse=True)))

            def pre(m, inp, st=st):
                self._sync()
                st["t"] = time.perf_counter()

            def post(m, inp, out, st=st):
                self._sync()
                st["ms"] += (time.perf_counter() - st.pop("t")) * 1e3
                st["calls"] += 1
                st["flops"] += module_forward_flops(m, inp, out)

            self.handles += [mod.register_forward_pre_hook(pre), mod.register_forward_hook(post)]
        self.started = True

    def stop(self):
        for h in self.handles:
            h.remove()
        self.handles, self.started = [], False

    def totals(self):
        """name -> flops including all descendants."""
        tot = {n: s["flops"] for n, s in self.stats.items()}
        for n in sorted(self.stats, key=lambda k: -k.count(".")):
            if n:
                parent = n.rsplit(".", 1)[0] if "." in n else ""
                tot[parent] += tot[n]
        return tot

    def report(self) -> str:
        tot = self.totals()
        root = dict(self.stats.get("", dict(params=0, ms=0.0)))
        if not root["ms"]:                 # a pipeline stage calls its layers one by one, never the container
            root["ms"] = sum(s["ms"] for n, s in self.stats.items() if n and "." not in n)
        lines = ["-" * 26 + " flops profiler " + "-" * 26,
                 f"profile step:                 {self.profile_step}",
                 f"parameters on this rank:      {root['params'] / 1e6:.3f} M",
                 f"forward FLOPs on this rank:   {tot.get('', 0.0) / 1e9:.3f} G",
                 f"forward latency:              {root['ms']:.3f} ms"]
        if root["ms"] > 0:
            lines.append(f"forward FLOP/s on this rank:  {tot.get('', 0.0) / root['ms'] / 1e9:.3f} T")
        depth_of = lambda n: 0 if n == "" else n.count(".") + 1
        max_depth = max(depth_of(n) for n in self.stats) if self.stats else 0
        upto = max_depth if self.module_depth < 0 else min(self.module_depth, max_depth)
        for d in range(1, upto + 1):
            rows = [(n, s) for n, s in self.stats.items() if depth_of(n) == d and s["calls"]]
            if not rows:
                continue
            lines.append(f"depth {d}:")
            for key, fmt in (("params", lambda s, n: f"{s['params'] / 1e6:.3f} M"),
                             ("flops", lambda s, n: f"{tot[n] / 1e9:.3f} GFLOPs"),
                             ("ms", lambda s, n: f"{s['ms']:.3f} ms")):
                val = (lambda n, s: tot[n]) if key == "flops" else (lambda n, s: s[key])
                top = sorted(rows, key=lambda r: -val(*r))[: self.top_modules]
                lines.append(f"    top {key}: " + ", ".join(f"{n} ({s['cls']}) {fmt(s, n)}" for n, s in top))
        if self.detailed:
            lines.append("per module (params, forward FLOPs incl. children, latency, calls):")
            for n, s in self.stats.items():
                if s["calls"] and (self.module_depth < 0 or depth_of(n) <= self.module_depth):
                    lines.append(f"  {'  ' * depth_of(n)}{n or '<model>'} [{s['cls']}]: {s['params'] / 1e6:.3f} M, "
                                 f"{tot[n] / 1e9:.3f} G, {s['ms']:.3f} ms, {s['calls']}x")
        return "\n".join(lines) + "\n"

    # engine hooks ---------------------------------------------------------------------------------
    def before_forward(self, global_step):
        if global_step == self.profile_step and not self.started and not self.stats:
            self.start()

    def after_step(self, global_step):
        if self.started:
            self.stop()
            text = self.report()
            if _rank() == 0:
                if self.output_file:
                    with open(self.output_file, "w") as f:
                        f.write(text)
                else:
                    print(text, flush=True)
            return text
        return None


# ---------------------------------------------------------------------------------------- comms logger
def _bus_factor(op: str, n: int) -> float:
    """Bus bandwidth / algorithm bandwidth for a ring or switch collective over ``n`` ranks."""
    if n <= 1:
        return 1.0
    if "all_reduce" in op:
        return 2.0 * (n - 1) / n
    if any(k in op for k in ("all_gather", "reduce_scatter", "all_to_all")):
        return (n - 1) / n
    return 1.0


def _message_bytes(op, args, kwargs, world):
    ts = [a for a in list(args) + list(kwargs.values()) if torch.is_tensor(a)]
    lists = [a for a in list(args) + list(kwargs.values()) if isinstance(a, (list, tuple)) and a and torch.is_tensor(a[0])]
    if op in ("all_gather", "reduce_scatter") and lists:
        return sum(t.numel() * t.element_size() for t in lists[0])
    if op in ("all_gather_into_tensor", "reduce_scatter_tensor") and ts:
        return max(t.numel() * t.element_size() for t in ts)           # the full (gathered / unreduced) buffer
    if ts:
        return ts[0].numel() * ts[0].element_size()
    return 0


class CommsLogger:
    OPS = ("all_reduce", "all_gather", "all_gather_into_tensor", "reduce_scatter", "reduce_scatter_tensor",
           "all_to_all_single", "broadcast", "reduce", "barrier", "send", "recv")

    def __init__(self, enabled=True, verbose=False, prof_all=True, debug=False, prof_ops=None):
        self.enabled, self.verbose, self.prof_all, self.debug = bool(enabled), bool(verbose), bool(prof_all), bool(debug)
        self.prof_ops = list(prof_ops or [])
        self.records = defaultdict(lambda: defaultdict(lambda: [0, 0.0, 1]))      # op -> bytes -> [count, ms, ranks]
        self._saved = {}

    @classmethod
    def from_args(cls, neox_args):
        cfg = getattr(neox_args, "comms_logger", None) or {}
        if not cfg.get("enabled"):
            return None
        return cls(**{k: cfg[k] for k in ("enabled", "verbose", "prof_all", "debug", "prof_ops") if k in cfg})

    def wants(self, op):
        return self.enabled and (self.prof_all or op in self.prof_ops)

    @contextlib.contextmanager
    def observe(self, op, nbytes, ranks=1, cuda=False, caller=None):
        """Time one collective: used by the wrappers below and by this framework's own NVLink collectives."""
        if not self.wants(op.split("[")[0]):
            yield
            return
        if cuda:
            torch.cuda.synchronize()
        t = time.perf_counter()
        try:
            yield
        finally:
            if cuda:
                torch.cuda.synchronize()
            ms = (time.perf_counter() - t) * 1e3
            rec = self.records[op][int(nbytes)]
            rec[0] += 1
            rec[1] += ms
            rec[2] = ranks
            if self.verbose and _rank() == 0:
                gbs = nbytes / max(ms, 1e-9) / 1e6
                where = f" | caller: {caller}" if (self.debug and caller) else ""
                print(f"comm op: {op} | time (ms): {ms:.3f} | msg size: {_fmt_bytes(nbytes)} | "
                      f"algbw (GB/s): {gbs:.2f} | busbw (GB/s): {gbs * _bus_factor(op, ranks):.2f}{where}", flush=True)

    def _wrap(self, name, fn):
        def wrapped(*args, **kwargs):
            group = kwargs.get("group", None)
            try:
                n = dist.get_world_size(group) if dist.is_initialized() else 1
            except Exception:  # noqa: BLE001 - not a member of the group: nothing to time
                return fn(*args, **kwargs)
            t0 = next((a for a in list(args) + list(kwargs.values()) if torch.is_tensor(a)), None)
            caller = sys._getframe(1).f_code.co_name if self.debug else None
            with self.observe(name, _message_bytes(name, args, kwargs, n), n, cuda=bool(t0 is not None and t0.is_cuda),
                              caller=caller):
                work = fn(*args, **kwargs)
                if kwargs.get("async_op") and work is not None:
                    work.wait()                      # a timed call is a finished call
            return work
        wrapped.neox_comms_wrapper = True
        wrapped.__name__ = name
        return wrapped

    def install(self):
        """Replace the ``torch.distributed`` entry points by timing wrappers (undone by `uninstall`)."""
        if self._saved or not self.enabled:
            return self
        for name in self.OPS:
            fn = getattr(dist, name, None)
            if fn is not None:
                self._saved[name] = fn
                setattr(dist, name, self._wrap(name, fn))
        from ..comm import collectives
        collectives.set_observer(self)
        return self

    def uninstall(self):
        for name, fn in self._saved.items():
            setattr(dist, name, fn)
        self._saved = {}
        from ..comm import collectives
        collectives.set_observer(None)

    def summary(self) -> str:
        head = f"{'comm. op':<32}{'message size':>14}{'count':>8}{'total (ms)':>13}{'avg (ms)':>11}" \
               f"{'algbw (GB/s)':>14}{'busbw (GB/s)':>14}"
        lines = [head]
        for op in sorted(self.records):
            for nbytes in sorted(self.records[op]):
                c, ms, n = self.records[op][nbytes]
                avg = ms / max(1, c)
                gbs = nbytes / max(avg, 1e-9) / 1e6
                lines.append(f"{op:<32}{_fmt_bytes(nbytes):>14}{c:>8}{ms:>13.2f}{avg:>11.3f}{gbs:>14.2f}"
                             f"{gbs * _bus_factor(op, n):>14.2f}")
        return "\n".join(lines) + "\n"

    def log_summary(self, out=None):
        text = self.summary()
        if _rank() == 0:
            print(text, file=out or sys.stdout, flush=True)
        return text


def _fmt_bytes(n):
    n = float(n)
    for unit in ("B", "KB", "MB", "GB"):
        if n < 1024 or unit == "GB":
            return f"{n:.2f} {unit}" if unit != "B" else f"{int(n)} B"
        n /= 1024


def dump_state(engine, out=None):
    """``dump_state: true``: the engine's effective settings, printed once on rank 0 after it is built."""
    if _rank() != 0:
        return None
    a = engine.neox_args
    rows = OrderedDict(
        zero_stage=engine.zero_stage, precision=a.precision, gradient_accumulation_steps=engine.gradient_accumulation_steps,
        train_batch_size=a.train_batch_size, train_micro_batch_size_per_gpu=a.train_micro_batch_size_per_gpu,
        gradient_clipping=engine.gradient_clipping, loss_scale=engine.loss_scaler.cur_scale,
        flat_groups=[dict(numel=g.numel(), dp_size=g.dp_size, dtype=str(g.params[0].dtype) if g.params else None)
                     for g in engine.groups],
        optimizer=type(engine.optimizer).__name__ if engine.optimizer is not None else None,
        lr_scheduler=type(engine.lr_scheduler).__name__ if engine.lr_scheduler is not None else None,
        pipeline_stages=getattr(engine, "num_stages", 1), comm_mode=_comm_mode())
    text = "engine state:\n" + "".join(f"  {k:.<40} {v}\n" for k, v in rows.items())
    print(text, file=out or sys.stdout, flush=True)
    return text


def _comm_mode():
    from ..comm import collectives
    return collectives.get_mode()
