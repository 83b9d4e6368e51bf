"""Maximal-update parametrisation (muP) for the NeoX model family, self-contained.

The reference delegates this to the external ``mup`` package (megatron/training.py:73-170,932-947,
1049-1090; megatron/model/init_functions.py:25-60; megatron/mup_substitute.py).  This module provides the
parts of it that training needs, stated directly:

* **base shapes**: the shapes of a *base* model and of a *delta* model (``hidden_size * mup_width_scale``)
  tell which dimensions of every parameter grow with width ("infinite" dimensions) and what their base
  size is.  ``make_base_shapes`` writes them to ``<base_shapes_file>.<rank>`` (YAML); ``set_base_shapes``
  attaches an :class:`InfShape` to every parameter of the target model.
* **width multiplier** of a parameter = current / base size of its fan-in dimension (two infinite
  dimensions: hidden x hidden matrices) or of its single infinite dimension (embeddings, biases, norms).
* **initialisation**: matrix-like weights are re-scaled by ``width_mult ** -0.5`` (what ``mup.init.normal_``
  does to the standard deviation); the read-out layer is rescaled by ``width_mult ** 0.5`` and divides its
  input by ``width_mult`` in the forward pass (MuReadout).
* **optimiser** (MuAdam / MuSGD): per-parameter learning-rate multipliers, carried as ``param.lr_mult`` /
  ``param.wd_mult`` and applied by the flat-buffer engine inside its fused update.
* **coordinate check**: mean absolute activation of every module over a few training steps for a range of
  widths, with and without muP; written as JSON (and plotted when matplotlib is importable).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, List, Optional

import torch
import yaml


class InfDim:
    """One dimension of a parameter: ``base`` is its size in the base model, or None when the dimension does
    not grow with width."""

    def __init__(self, base: Optional[int], dim: int):
        self.base, self.dim = base, int(dim)

    def isinf(self) -> bool:
        return self.base is not None

    def width_mult(self) -> float:
        return self.dim / self.base if self.base is not None else 1.0

    def __repr__(self):
        return f"InfDim({self.base}, {self.dim})"


class InfShape:
    def __init__(self, dims: List[InfDim]):
        self.dims = list(dims)
        if self.ninf() > 2:
            raise ValueError(f"muP: a parameter with {self.ninf()} width-dependent dimensions is not supported: {dims}")

    def ninf(self) -> int:
        return sum(d.isinf() for d in self.dims)

    def main_idx(self) -> Optional[int]:
        """Index of the dimension that defines the width multiplier: the only infinite one, or the fan-in
        (second) one of a [fan_out, fan_in, ...] matrix."""
        inf = [i for i, d in enumerate(self.dims) if d.isinf()]
        if not inf:
            return None
        return inf[0] if len(inf) == 1 else inf[1]

    def width_mult(self) -> float:
        i = self.main_idx()
        return 1.0 if i is None else self.dims[i].width_mult()

    def fanin_fanout_mult_ratio(self) -> float:
        inf = [d for d in self.dims if d.isinf()]
        assert len(inf) == 2, "fan-in / fan-out ratio is defined for matrix-like parameters only"
        return inf[1].width_mult() / inf[0].width_mult()

    def __repr__(self):
        return f"InfShape({self.dims})"


# ------------------------------------------------------------------------------------------ base shapes
def get_shapes(model: torch.nn.Module) -> Dict[str, List[int]]:
    return {name: list(p.shape) for name, p in model.named_parameters()}


def make_base_shapes(base_shapes: Dict[str, List[int]], delta_shapes: Dict[str, List[int]],
                     savefile: Optional[str] = None) -> Dict[str, List[Optional[int]]]:
    """Per parameter, the base size of every dimension that differs between the base and the delta model
    (None for dimensions that do not depend on width)."""
    if base_shapes.keys() != delta_shapes.keys():
        raise ValueError("muP: the base and delta models have different parameters")
    out = {}
    for name, b in base_shapes.items():
        d = delta_shapes[name]
        if len(b) != len(d):
            raise ValueError(f"muP: {name} has rank {len(b)} in the base model and {len(d)} in the delta model")
        out[name] = [bi if bi != di else None for bi, di in zip(b, d)]
    if savefile is not None:
        os.makedirs(os.path.dirname(os.path.abspath(savefile)), exist_ok=True)
        with open(savefile, "w") as f:
            yaml.safe_dump(out, f)
    return out


def load_base_shapes(path: str) -> Dict[str, List[Optional[int]]]:
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"muP base-shapes file {path} not found: run once with `save_base_shapes: true` (same parallel "
            f"layout) to create it")
    with open(path) as f:
        return yaml.safe_load(f)


def set_base_shapes(model: torch.nn.Module, base) -> torch.nn.Module:
    """Attach ``.infshape`` to every parameter.  ``base``: a base-shapes dict or the path of a saved one."""
    shapes = load_base_shapes(base) if isinstance(base, str) else base
    for name, p in model.named_parameters():
        if name not in shapes:
            raise KeyError(f"muP: parameter {name} is missing from the base shapes")
        b = shapes[name]
        if len(b) != p.dim():
            raise ValueError(f"muP: {name} has rank {p.dim()}, base shapes say {len(b)}")
        p.infshape = InfShape([InfDim(bi, di) for bi, di in zip(b, p.shape)])
    return model


# ------------------------------------------------------------------------------------------ init + optimiser
def lr_multiplier(infshape: InfShape, optimizer: str) -> float:
    """MuAdam: matrix-like lr / width_mult.  MuSGD: vector-like lr * width_mult, matrix-like lr / (fan-in mult /
    fan-out mult)."""
    n = infshape.ninf()
    if optimizer == "adam":
        return 1.0 / infshape.width_mult() if n == 2 else 1.0
    if optimizer == "sgd":
        if n == 1:
            return infshape.width_mult()
        if n == 2:
            return 1.0 / infshape.fanin_fanout_mult_ratio()
        return 1.0
    raise ValueError(f"muP supports the adam and sgd optimizers, got {optimizer}")


def apply_mup(model: torch.nn.Module, optimizer: str = "adam", reinit: bool = True) -> torch.nn.Module:
    """After ``set_base_shapes``: rescale the initialisation, mark the read-out layers and set the
    per-parameter learning-rate / weight-decay multipliers the engine applies."""
    readout = set()
    for m in model.modules():
        if getattr(m, "mup_rescale_parameters", False) and hasattr(m, "weight"):
            wm = m.weight.infshape.width_mult()
            m.width_mult_value = wm          # forward divides the read-out input by this
            m.use_mup = True
            if reinit and not getattr(m, "_has_rescaled_params", False):
                with torch.no_grad():
                    m.weight.mul_(wm ** 0.5)
                    if getattr(m, "bias", None) is not None:
                        m.bias.mul_(wm ** 0.5)
                m._has_rescaled_params = True
            readout.add(id(m.weight))
    for name, p in model.named_parameters():
        shp = p.infshape
        if reinit and shp.ninf() == 2 and id(p) not in readout:
            with torch.no_grad():
                p.mul_(shp.width_mult() ** -0.5)
        p.lr_mult = lr_multiplier(shp, optimizer)
        # coupled decay: keep lr * weight_decay of matrix-like weights independent of width
        p.wd_mult = shp.width_mult() if (optimizer == "adam" and shp.ninf() == 2) else 1.0
    return model


# ------------------------------------------------------------------------------------------ coordinate check
def record_coords(records: list, width: int, name: str, step: int) -> Callable:
    """Forward hook appending the mean absolute value of a module's output."""
    def hook(_module, _inp, out):
        t = out[0] if isinstance(out, (tuple, list)) else out
        if torch.is_tensor(t) and t.is_floating_point():
            records.append({"width": width, "module": name, "t": step, "l1": float(t.detach().float().abs().mean())})
    return hook


def get_coord_data(models: Dict[int, Callable[[], object]], train_one_step: Callable[[object], None],
                   nsteps: int = 3, nseeds: int = 1, filter_module_by_name: Optional[Callable[[str], bool]] = None):
    """For every width build the model (``models[width]()`` returns it), train ``nsteps`` steps with
    ``train_one_step(model)`` and record every module's output scale at every step."""
    records = []
    for seed in range(nseeds):
        torch.manual_seed(seed)
        for width, make in models.items():
            model = make()
            net = getattr(model, "module", model)
            for step in range(1, nsteps + 1):
                handles = []
                for name, module in net.named_modules():
                    if not name or (filter_module_by_name and not filter_module_by_name(name)):
                        continue
                    handles.append(module.register_forward_hook(record_coords(records, width, name, step)))
                train_one_step(model)
                for h in handles:
                    h.remove()
            del model, net
    return records


def growth_exponents(records) -> Dict[str, float]:
    """Least-squares slope of log(l1) against log(width) at the last recorded step, per module: near 0 for a
    width-stable parametrisation."""
    import math
    last = max(r["t"] for r in records)
    by_mod: Dict[str, list] = {}
    for r in records:
        if r["t"] == last and r["l1"] > 0:
            by_mod.setdefault(r["module"], []).append((math.log(r["width"]), math.log(r["l1"])))
    out = {}
    for name, pts in by_mod.items():
        if len({x for x, _ in pts}) < 2:
            continue
        n = len(pts)
        mx, my = sum(x for x, _ in pts) / n, sum(y for _, y in pts) / n
        den = sum((x - mx) ** 2 for x, _ in pts)
        out[name] = sum((x - mx) * (y - my) for x, y in pts) / den
    return out


def save_coord_data(records, path_stem: str):
    """``<stem>.json`` always; ``<stem>.jpg`` (one panel per step, l1 against width per module) when matplotlib
    is importable."""
    with open(path_stem + ".json", "w") as f:
        json.dump(records, f)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return
    steps = sorted({r["t"] for r in records})
    fig, axes = plt.subplots(1, len(steps), figsize=(5 * len(steps), 4), squeeze=False)
    for ax, t in zip(axes[0], steps):
        mods = sorted({r["module"] for r in records})
        for m in mods:
            pts = sorted((r["width"], r["l1"]) for r in records if r["t"] == t and r["module"] == m)
            if pts:
                ax.plot([p[0] for p in pts], [p[1] for p in pts], marker="o", linewidth=0.8)
        ax.set_xscale("log", base=2)
        ax.set_yscale("log")
        ax.set_title(f"t={t}")
        ax.set_xlabel("width")
        ax.set_ylabel("l1")
    fig.tight_layout()
    fig.savefig(path_stem + ".jpg")
    plt.close(fig)
