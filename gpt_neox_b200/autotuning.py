"""Autotuning of the batch / ZeRO keys: short profiled trial runs, then the best configuration.

The reference forwards ``--autotuning tune|run`` to the DeepSpeed autotuner (deepy.py:22-37,
megatron/neox_arguments/arguments.py:95-101,497-505: the five keys ``train_batch_size``,
``train_micro_batch_size_per_gpu``, ``gradient_accumulation_steps``, ``zero_optimization`` and
``autotuning`` of a returned ``--deepspeed_config`` file override the NeoX config;
configs/autotuning_configs/*.json are the shipped search spaces).  Here the tuner is part of the
framework:

* the **search space** is the list of ZeRO stages (``zero_optimization.stage`` may be a list) times the
  micro-batch sizes that a memory model of the job says can fit in one GPU's HBM
  (`memory_per_gpu`: parameters, gradients and optimizer state by stage, activations per micro-batch with
  or without activation checkpointing, the logits of the last stage);
* an **experiment** is the user's own script started through the ordinary launcher with an override
  file, stopped by the training loop after ``end_profile_step`` steps (`ProfileWindow`), which leaves the
  measured throughput in ``metric_path``; a run that dies (out of memory) leaves no file and prunes the
  larger micro-batches of its stage;
* tuner types ``gridsearch``, ``random`` and ``model_based`` (per stage, micro-batch sizes in rising order,
  stopped after ``tuner_early_stopping`` trials without an improvement);
* results go to ``autotuning_results/`` (one JSON per experiment, ``summary.txt``,
  ``ds_config_optimal.json``); ``--autotuning run`` then starts the job with the optimal file.
"""
from __future__ import annotations

import copy
import json
import math
import os
import random
import time
from typing import Callable, Dict, List, Optional

METRICS = ("throughput", "latency", "flops")
DEFAULTS = dict(enabled=False, fast=True, metric="throughput", start_profile_step=3, end_profile_step=5,
                tuner_type="gridsearch", tuner_early_stopping=5, tuner_num_trials=50, results_dir="autotuning_results",
                exps_dir="autotuning_exps", overwrite=True, max_train_batch_size=None,
                min_train_micro_batch_size_per_gpu=1, max_train_micro_batch_size_per_gpu=1024,
                num_tuning_micro_batch_sizes=3, mp_size=1, arg_mappings=None, hbm_bytes=180e9, hbm_fraction=0.9)


def settings(ds_config: dict) -> dict:
    """The ``autotuning`` block of a config with the defaults filled in."""
    out = dict(DEFAULTS)
    out.update(ds_config.get("autotuning") or {})
    if out["metric"] not in METRICS:
        raise ValueError(f"autotuning metric must be one of {METRICS}, not {out['metric']!r}")
    return out


# ---------------------------------------------------------------------------------------- memory model
def model_info(cfg: dict) -> dict:
    """Sizes the memory model needs, from a NeoX config dict (dashes or underscores in the keys)."""
    c = {k.replace("-", "_"): v for k, v in cfg.items()}
    h, L = int(c.get("hidden_size", 0)), int(c.get("num_layers", 0))
    ffn = int(c.get("intermediate_size") or 4 * h)
    gated = str(c.get("activation", "gelu")) in ("swiglu", "geglu", "reglu")
    vocab = int(c.get("padded_vocab_size") or c.get("vocab_size") or 50432)
    heads = int(c.get("num_attention_heads", 1) or 1)
    kv = int(c.get("num_kv_heads") or heads)
    attn = h * h * (2 + 2 * kv / heads)
    mlp = (3 if gated else 2) * h * ffn
    experts = int(c.get("moe_num_experts", 1) or 1)
    per_layer = attn + mlp * experts + 4 * h
    tied = not c.get("no_weight_tying", False)
    return dict(hidden=h, layers=L, seq=int(c.get("seq_length", 2048)), vocab=vocab,
                params=int(L * per_layer + vocab * h * (1 if tied else 2)),
                tp=int(c.get("model_parallel_size", 1) or 1), pp=int(c.get("pipe_parallel_size", 1) or 1),
                checkpoint=bool(c.get("checkpoint_activations", False)),
                sequence_parallel=bool(c.get("sequence_parallel", False)))


def memory_per_gpu(info: dict, stage: int, micro_batch: int, dp: int) -> float:
    """Bytes one GPU holds for a step: bf16 parameters, fp32 gradient accumulators, fp32 master + two Adam
    moments (split over data parallel from stage 1 on, gradients from stage 2 on), plus activations."""
    shard = info["params"] / (info["tp"] * info["pp"])
    dp = max(1, dp)
    weights = 2.0 * shard
    grads = 4.0 * shard / (dp if stage >= 2 else 1)
    optim = 12.0 * shard / (dp if stage >= 1 else 1)
    s, b, h = info["seq"], micro_batch, info["hidden"]
    layers = max(1, math.ceil(info["layers"] / info["pp"]))
    tp_act = info["tp"]
    if info["checkpoint"]:                      # one saved input per layer + one layer live
        per_layer = 2.0 * s * b * h / (tp_act if info["sequence_parallel"] else 1)
        act = layers * per_layer + 34.0 * s * b * h / tp_act
    else:                                       # flash attention: no s^2 term
        act = layers * 34.0 * s * b * h / tp_act
    in_flight = min(info["pp"], 4) if info["pp"] > 1 else 1
    logits = 6.0 * s * b * info["vocab"] / info["tp"]
    return weights + grads + optim + act * in_flight + logits


def max_micro_batch(info: dict, stage: int, dp: int, budget: float, cap: int) -> int:
    """Largest power-of-two micro-batch size whose modelled footprint stays inside ``budget`` bytes (0: none)."""
    best, b = 0, 1
    while b <= cap:
        if memory_per_gpu(info, stage, b, dp) > budget:
            break
        best, b = b, b * 2
    return best


# ---------------------------------------------------------------------------------------- search space
def _stages(ds_config: dict) -> List[int]:
    z = (ds_config.get("zero_optimization") or {}).get("stage", 0)
    stages = list(z) if isinstance(z, (list, tuple)) else [int(z)]
    # stage 3 (parameter partitioning) is not offered together with tensor / pipeline parallelism
    return [int(s) for s in stages if int(s) in (0, 1, 2)] or [0]


def build_space(ds_config: dict, info: dict, world_size: int) -> List[dict]:
    """Experiments as override dicts of the five tuned keys, grouped by stage, micro-batch size rising."""
    st = settings(ds_config)
    dp = max(1, world_size // (info["tp"] * info["pp"]))
    budget = st["hbm_bytes"] * st["hbm_fraction"]
    exps = []
    for stage in _stages(ds_config):
        top = max_micro_batch(info, stage, dp, budget, int(st["max_train_micro_batch_size_per_gpu"]))
        if top == 0:
            continue
        sizes, b = [], top
        while b >= max(1, int(st["min_train_micro_batch_size_per_gpu"])) and len(sizes) < int(st["num_tuning_micro_batch_sizes"]):
            sizes.append(b)
            b //= 2
        for mbs in sorted(sizes):
            gas = int(ds_config.get("gradient_accumulation_steps") or 1)
            if st["max_train_batch_size"]:
                gas = max(1, int(st["max_train_batch_size"]) // (mbs * dp))
            zero = copy.deepcopy(ds_config.get("zero_optimization") or {})
            zero["stage"] = stage
            exps.append(dict(name=f"z{stage}_mbs{mbs}_gas{gas}", train_micro_batch_size_per_gpu=mbs,
                             gradient_accumulation_steps=gas, train_batch_size=mbs * gas * dp,
                             zero_optimization=zero))
    return exps


# ---------------------------------------------------------------------------------------- tuner
class Autotuner:
    """Runs experiments through ``run_experiment(overrides, exp_dir) -> metrics dict or None`` (None: the
    run failed, which is read as out of memory) and keeps the best by the configured metric."""

    def __init__(self, ds_config: dict, neox_config: dict, world_size: int,
                 run_experiment: Callable[[dict, str], Optional[dict]], seed: int = 0, log=print):
        self.ds_config = ds_config
        self.st = settings(ds_config)
        self.info = model_info(neox_config)
        self.world_size = world_size
        self.run_experiment = run_experiment
        self.records: List[dict] = []
        self.rng = random.Random(seed)
        self.log = log

    def _score(self, m: dict) -> float:
        v = float(m[self.st["metric"]])
        return -v if self.st["metric"] == "latency" else v

    def _order(self, exps: List[dict]) -> List[dict]:
        if self.st["tuner_type"] == "random":
            exps = list(exps)
            self.rng.shuffle(exps)
        return exps

    def tune(self) -> Optional[dict]:
        exps = self._order(build_space(self.ds_config, self.info, self.world_size))
        exps = exps[: int(self.st["tuner_num_trials"])]
        os.makedirs(self.st["results_dir"], exist_ok=True)
        os.makedirs(self.st["exps_dir"], exist_ok=True)
        oom_at: Dict[int, int] = {}          # stage -> smallest micro-batch size that failed
        best, since_best, stage_since = None, 0, {}
        for exp in exps:
            stage, mbs = exp["zero_optimization"]["stage"], exp["train_micro_batch_size_per_gpu"]
            if stage in oom_at and mbs >= oom_at[stage]:
                self.records.append(dict(exp, status="pruned"))
                continue
            if self.st["tuner_type"] == "model_based" and stage_since.get(stage, 0) >= int(self.st["tuner_early_stopping"]):
                self.records.append(dict(exp, status="early_stopped"))
                continue
            if self.st["tuner_type"] != "model_based" and since_best >= int(self.st["tuner_early_stopping"]):
                self.records.append(dict(exp, status="early_stopped"))
                continue
            exp_dir = os.path.join(self.st["exps_dir"], exp["name"])
            os.makedirs(exp_dir, exist_ok=True)
            t0 = time.time()
            metrics = self.run_experiment(exp, exp_dir)
            rec = dict(exp, seconds=round(time.time() - t0, 2))
            if metrics is None:
                rec["status"] = "failed"
                oom_at[stage] = min(mbs, oom_at.get(stage, mbs))
            else:
                rec.update(status="ok", metrics=metrics)
                if best is None or self._score(metrics) > self._score(best["metrics"]):
                    best, since_best, stage_since[stage] = rec, 0, 0
                else:
                    since_best += 1
                    stage_since[stage] = stage_since.get(stage, 0) + 1
            self.records.append(rec)
            with open(os.path.join(self.st["results_dir"], exp["name"] + ".json"), "w") as f:
                json.dump(rec, f, indent=1)
            self.log(f"autotuning: {exp['name']}: {rec['status']}" +
                     (f" {self.st['metric']}={metrics[self.st['metric']]:.4g}" if metrics else ""))
        self.best = best
        self.write_summary()
        return best

    def optimal_config(self) -> Optional[dict]:
        if getattr(self, "best", None) is None:
            return None
        cfg = copy.deepcopy(self.ds_config)
        for k in ("train_batch_size", "train_micro_batch_size_per_gpu", "gradient_accumulation_steps", "zero_optimization"):
            cfg[k] = self.best[k]
        cfg.pop("autotuning", None)
        return cfg

    def write_summary(self) -> str:
        d = self.st["results_dir"]
        lines = [f"{'experiment':<28}{'status':<16}{self.st['metric']:>14}"]
        for r in self.records:
            v = r.get("metrics", {}).get(self.st["metric"])
            lines.append(f"{r['name']:<28}{r['status']:<16}{(f'{v:.4g}' if v is not None else '-'):>14}")
        if getattr(self, "best", None) is not None:
            lines.append(f"best: {self.best['name']}")
            with open(os.path.join(d, "ds_config_optimal.json"), "w") as f:
                json.dump(self.optimal_config(), f, indent=1)
        else:
            lines.append("best: none (no experiment finished)")
        text = "\n".join(lines) + "\n"
        with open(os.path.join(d, "summary.txt"), "w") as f:
            f.write(text)
        return text


# ---------------------------------------------------------------------------------------- training side
class ProfileWindow:
    """What the training loop does during an experiment: time the steps from ``start_profile_step`` to
    ``end_profile_step`` (device-synchronised on both sides), have rank 0 write the metrics to
    ``metric_path`` and tell the loop to stop."""

    def __init__(self, start_step, end_step, metric_path, samples_per_step, flops_per_step=0.0):
        self.start_step, self.end_step = int(start_step), int(end_step)
        if self.end_step <= self.start_step:
            raise ValueError("autotuning: end_profile_step must be larger than start_profile_step")
        self.metric_path = metric_path
        self.samples_per_step = samples_per_step
        self.flops_per_step = flops_per_step
        self.t0 = None

    @classmethod
    def from_args(cls, neox_args):
        at = getattr(neox_args, "autotuning", None) or {}
        if not at.get("enabled") or not at.get("metric_path"):
            return None
        st = dict(DEFAULTS)
        st.update(at)
        flops = 0.0
        try:
            from .obs.logging import get_flops
            flops = float(get_flops(neox_args, 1.0))            # per GPU and step
        except Exception:  # noqa: BLE001 - the flops metric is optional
            pass
        return cls(st["start_profile_step"], st["end_profile_step"], at["metric_path"], neox_args.train_batch_size,
                   flops)

    @staticmethod
    def _sync():
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def after_step(self, iteration: int, rank: int = 0) -> bool:
        """Call with the number of finished steps; True once the window has closed and the file is written."""
        if iteration == self.start_step:
            self._sync()
            self.t0 = time.perf_counter()
            return False
        if iteration >= self.end_step and self.t0 is not None:
            self._sync()
            dt = (time.perf_counter() - self.t0) / (iteration - self.start_step)
            metrics = dict(latency=dt, throughput=self.samples_per_step / dt, flops=self.flops_per_step / dt)
            if rank == 0:
                tmp = self.metric_path + ".tmp"
                with open(tmp, "w") as f:
                    json.dump(metrics, f)
                os.replace(tmp, self.metric_path)
            return True
        return False


# ---------------------------------------------------------------------------------------- launcher side
def _arg_value(argv: List[str], flag: str):
    for i, a in enumerate(argv):
        if a == flag and i + 1 < len(argv):
            return i + 1, argv[i + 1]
        if a.startswith(flag + "="):
            return i, a[len(flag) + 1:]
    return None, None


def _decode(raw: str) -> dict:
    import base64
    if os.path.exists(raw):
        with open(raw) as f:
            return json.load(f)
    return json.loads(base64.urlsafe_b64decode(raw).decode("utf-8"))


def run_from_launcher(mode: str, user_args: List[str], world_size: int, launch: Callable[[List[str]], int],
                      log=print) -> int:
    """``--autotuning tune|run`` of the launcher.  ``user_args`` carry ``--deepspeed_config`` (a file in this
    mode) and ``--megatron_config``; ``launch(user_args) -> exit code`` starts the job once."""
    pos, raw = _arg_value(user_args, "--deepspeed_config")
    if raw is None:
        raise ValueError("autotuning needs --deepspeed_config among the script arguments")
    ds_config = _decode(raw)
    _, mraw = _arg_value(user_args, "--megatron_config")
    neox_config = _decode(mraw) if mraw is not None else {}
    neox_config = dict(neox_config, **{k: v for k, v in ds_config.items() if k not in neox_config})

    def with_config(path):
        args = list(user_args)
        if args[pos].startswith("--deepspeed_config="):
            args[pos] = "--deepspeed_config=" + path
        else:
            args[pos] = path
        return args

    def run_experiment(exp, exp_dir):
        cfg = copy.deepcopy(ds_config)
        for k in ("train_batch_size", "train_micro_batch_size_per_gpu", "gradient_accumulation_steps", "zero_optimization"):
            cfg[k] = exp[k]
        metric_path = os.path.abspath(os.path.join(exp_dir, "metrics.json"))
        if os.path.exists(metric_path):
            os.remove(metric_path)
        cfg["autotuning"] = dict(settings(ds_config), enabled=True, metric_path=metric_path)
        path = os.path.abspath(os.path.join(exp_dir, "ds_config.json"))
        with open(path, "w") as f:
            json.dump(cfg, f, indent=1)
        rc = launch(with_config(path))
        if not os.path.exists(metric_path):
            log(f"autotuning: {exp['name']} left no metrics (exit code {rc})")
            return None
        with open(metric_path) as f:
            return json.load(f)

    tuner = Autotuner(ds_config, neox_config, world_size, run_experiment, log=log)
    best = tuner.tune()
    log(tuner.write_summary())
    if best is None:
        return 1
    if mode == "run":
        path = os.path.abspath(os.path.join(tuner.st["results_dir"], "ds_config_optimal.json"))
        return launch(with_config(path))
    return 0
