"""NeoXArgs: the one configuration object of the framework.

Same user surface as the reference (megatron/neox_arguments/arguments.py:125-1477): N YAML files
are merged (a key may appear in one file only, ``-`` and ``_`` are interchangeable), a few CLI
flags of ``deepy.py`` override them, values are type-checked against the schema table, derived
values are computed (GPU count, data-parallel size, the batch triple, precision dicts, ZeRO
mirrors, attention-type expansion) and the result travels to every rank as url-safe base64 JSON
of the non-default values (``--megatron_config``).  Built from ``schema.SCHEMA`` instead of twelve
hand-written dataclasses.
"""
from __future__ import annotations

import argparse
import base64
import copy
import json
import logging
import os
import shutil
import subprocess
import sys
from typing import Any

import yaml

from .schema import EXTENSIONS, REQUIRED, SCHEMA

ATTENTION_TYPE_CHOICES = ["global", "local", "sparse_fixed", "sparse_variable", "bigbird", "bslongformer",
                          "gmlp", "amlp", "flash", "rwkv", "mamba"]
ZERO_DEFAULTS = {"stage": 0, "allgather_partitions": True, "reduce_scatter": True,
                 "allgather_bucket_size": int(5e8), "overlap_comm": False, "reduce_bucket_size": int(5e8),
                 "contiguous_gradients": False}
OPT_DEFAULT = "Adam"
OPT_PARAMS_DEFAULTS = {"lr": 0.001, "betas": [0.9, 0.999], "eps": 1.0e-8, "weight_decay": 0,
                       "freeze_step": 400, "momentum": 0.0, "cuda_aware": False}
AUTOTUNING_ARGS = ("train_batch_size", "train_micro_batch_size_per_gpu", "gradient_accumulation_steps",
                   "zero_optimization", "autotuning")
DEFAULT_HOSTFILE = "/job/hostfile"

FIELDS: dict[str, tuple[str, str, Any]] = {}      # name -> (group, type, default)
for _g, _entries in SCHEMA.items():
    for _n, _t, _d in _entries:
        assert _n not in FIELDS, f"duplicate field {_n} in schema"
        FIELDS[_n] = (_g, _t, _d)


# ----------------------------------------------------------------------------------------------
# type grammar
# ----------------------------------------------------------------------------------------------
def _split_top(s: str) -> list[str]:
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch == "[":
            depth += 1
        elif ch == "]":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def type_ok(value, t: str) -> bool:
    """True if ``value`` conforms to the schema type ``t`` (None always passes)."""
    if value is None or t == "Any":
        return True
    if t == "bool":
        return isinstance(value, bool)
    if t == "int":
        return isinstance(value, int) and not isinstance(value, bool)
    if t == "float":
        return isinstance(value, (int, float)) and not isinstance(value, bool)
    if t == "str":
        return isinstance(value, str)
    if t == "dict":
        return isinstance(value, dict)
    if t == "list":
        return isinstance(value, (list, tuple))
    if t == "list_of_int":
        return isinstance(value, (list, tuple)) and all(type_ok(v, "int") for v in value)
    if t == "list_of_str":
        return isinstance(value, (list, tuple)) and all(isinstance(v, str) for v in value)
    if t.startswith("one_of["):
        choices = [c.strip().strip("'\"") for c in _split_top(t[len("one_of["):-1])]
        return isinstance(value, str) and value.lower() in [c.lower() for c in choices]
    if t.startswith("any_of["):
        return any(type_ok(value, x) for x in _split_top(t[len("any_of["):-1]))
    raise ValueError(f"unknown schema type {t}")


def expand_attention_types(attention_config, num_layers: int):
    """``[[["flash"], 32]]`` / ``[[["global","local"], "all"]]`` -> one type per layer
    (megatron/utils.py:326-353). A flat list of strings is taken as already expanded."""
    if all(isinstance(i, str) for i in attention_config):
        return list(attention_config)
    out = []
    for item in attention_config:
        if item[1] == "all":
            assert num_layers % len(item[0]) == 0, \
                f"Number of layers ({num_layers}) is not divisible by the length of pattern: {item[0]}"
            return list(item[0]) * (num_layers // len(item[0]))
        for _ in range(item[1]):
            out.extend(item[0])
    return out


def _git_hash():
    try:
        if shutil.which("git") is None:
            return None
        r = subprocess.run(["git", "describe", "--always"], capture_output=True, text=True,
                           cwd=os.path.dirname(os.path.abspath(__file__)), timeout=5)
        return r.stdout.strip() or None
    except Exception:
        return None


def _parse_hostfile(path, include="", exclude=""):
    """``host slots=N`` lines -> ordered {host: [slot ids]}, with the runner's include / exclude
    filters (``host1@host2:0,1`` syntax)."""
    pool = {}
    with open(path) as f:
        for line in f:
            line = line.split("#")[0].strip()
            if not line:
                continue
            host, _, rest = line.partition(" ")
            slots = 1
            for tok in rest.split():
                if tok.startswith("slots="):
                    slots = int(tok.split("=")[1])
            pool[host] = list(range(slots))

    def parse_filter(s):
        res = {}
        for part in filter(None, s.split("@")):
            host, _, ids = part.partition(":")
            res[host] = [int(i) for i in ids.split(",")] if ids else None
        return res
    if include:
        inc = parse_filter(include)
        pool = {h: (inc[h] if inc[h] is not None else pool[h]) for h in pool if h in inc}
    if exclude:
        exc = parse_filter(exclude)
        for h, ids in exc.items():
            if h in pool:
                if ids is None:
                    del pool[h]
                else:
                    pool[h] = [i for i in pool[h] if i not in ids]
        pool = {h: v for h, v in pool.items() if v}
    return pool


class NeoXArgs:
    """All arguments of a run. Construct with ``from_ymls`` / ``from_dict`` / ``consume_deepy_args``
    / ``consume_neox_args``; unknown keys raise ``TypeError`` as a dataclass would."""

    def __init__(self, **kwargs):
        unknown = [k for k in kwargs if k not in FIELDS]
        if unknown:
            raise TypeError(f"NeoXArgs got unexpected argument(s): {sorted(unknown)}")
        for name, (_g, _t, default) in FIELDS.items():
            object.__setattr__(self, name, copy.deepcopy(default))
        for k, v in kwargs.items():
            object.__setattr__(self, k, v)
        if self.git_hash is None:
            self.git_hash = _git_hash()
        self.__post_init__()

    # ------------------------------------------------------------------ construction
    def __post_init__(self):
        if not self.validate_keys():
            raise ValueError(self.__class__.__name__ + ".__post_init__() NeoXArgs keys cannot be validated")
        self.calculate_derived()
        if not self.validate_types():
            raise ValueError(self.__class__.__name__ + ".__post_init__() NeoXArgs types cannot be validated")
        if not self.validate_values():
            raise ValueError(self.__class__.__name__ + ".__post_init__() NeoXArgs values cannot be validated")

    @classmethod
    def from_ymls(cls, paths_to_yml_files, overwrite_values: dict | None = None):
        """Merge several YAML files; a key defined in two files is an error."""
        config: dict = {}
        config_files = {}
        for conf_file_name in paths_to_yml_files:
            with open(conf_file_name) as f:
                raw = f.read()
            conf = yaml.safe_load(raw) or {}
            for k, v in conf.items():
                key = k.replace("-", "_")
                if key in config:
                    raise ValueError(f"Conf file {conf_file_name} has the following duplicate keys with "
                                     f"previously loaded file: {key}")
                config[key] = v
            config_files[os.path.basename(conf_file_name)] = raw
        config["config_files"] = config_files
        if overwrite_values:
            for k, v in overwrite_values.items():
                config[k] = v
        return cls(**config)

    @classmethod
    def from_dict(cls, args_dict: dict):
        return cls(**{k.replace("-", "_"): v for k, v in args_dict.items()})

    @classmethod
    def consume_deepy_args(cls, input_args=None):
        """Parse the ``deepy.py`` command line: user script, config files and the overrides
        (megatron/neox_arguments/arguments.py:298-458)."""
        parser = argparse.ArgumentParser(description="GPT-NeoX Configuration", allow_abbrev=False)
        group = parser.add_argument_group(title="Training Configuration")
        group.add_argument("user_script", type=str,
                           help="User script to launch, followed by any required arguments.")
        group.add_argument("--conf_dir", "-d", type=str, default=None,
                           help="Directory to prefix to all configuration file paths")
        group.add_argument("conf_file", type=str, nargs="+",
                           help="Configuration file path(s), merged in order.")
        group = parser.add_argument_group(title="Weights and Biases monitoring args")
        group.add_argument("--wandb_group", type=str, default=None)
        group.add_argument("--wandb_run_name", type=str, default=None)
        group.add_argument("--wandb_team", type=str, default=None)
        group = parser.add_argument_group(title="Eval args")
        group.add_argument("--eval_tasks", type=str, nargs="+", default=None)
        group.add_argument("--iteration", type=int, default=None)
        group.add_argument("--eval_results_prefix", type=str, default=None)
        group = parser.add_argument_group(title="Generation args")
        group.add_argument("-i", "--sample_input_file", type=str, default=None)
        group.add_argument("-o", "--sample_output_file", type=str, default=None)
        group = parser.add_argument_group(title="Launcher args")
        group.add_argument("-H", "--hostfile", type=str)
        group = parser.add_argument_group(title="Autotuning")
        group.add_argument("--autotuning", type=str, default=None, choices=("tune", "run"))
        args_parsed = parser.parse_args(input_args)

        conf_files = args_parsed.conf_file
        if args_parsed.conf_dir:
            conf_files = [os.path.join(args_parsed.conf_dir, f) for f in conf_files]
        conf_files = [(cf if (cf.endswith(".yml") or cf.endswith(".json")) else cf + ".yml") for cf in conf_files]

        overwrite_values = {}
        for k, v in vars(args_parsed).items():
            if k == "autotuning" and v is not None:
                overwrite_values["autotuning_run"] = v
            elif k not in ("conf_dir", "conf_file") and v is not None:
                overwrite_values[k] = v
        neox_args = cls.from_ymls(paths_to_yml_files=conf_files, overwrite_values=overwrite_values)
        if neox_args.use_wandb:
            try:
                import wandb  # noqa: F401
                neox_args.wandb_group = (neox_args.wandb_group or "run") + "_" + os.urandom(4).hex()
            except ModuleNotFoundError:
                pass
        return neox_args

    @classmethod
    def consume_neox_args(cls, overwrite_values=None, input_args=None):
        """Per-rank entry: rebuild the args from ``--megatron_config`` (base64 JSON)."""
        parser = argparse.ArgumentParser(description="GPT-NeoX Configuration", allow_abbrev=False)
        parser.add_argument("--megatron_config", type=str, default=None,
                            help="Megatron configuration dict, base64-encoded JSON or a path to a JSON file")
        parser.add_argument("--deepspeed_config", type=str, default=None,
                            help="Only needed during autotuning: overrides the tuned batch / ZeRO keys")
        parser.add_argument("--local_rank", type=int, default=None)
        args_parsed, _ = parser.parse_known_args(input_args)
        cfg = args_parsed.megatron_config
        if cfg is None:
            raise ValueError("--megatron_config is required")
        if os.path.exists(cfg):
            with open(cfg) as f:
                megatron_config = json.load(f)
        else:
            megatron_config = json.loads(base64.urlsafe_b64decode(cfg).decode("utf-8"))
        if args_parsed.deepspeed_config is not None:
            raw = args_parsed.deepspeed_config
            ds = json.load(open(raw)) if os.path.exists(raw) else json.loads(
                base64.urlsafe_b64decode(raw).decode("utf-8"))
            for k in AUTOTUNING_ARGS:
                if k in ds:
                    megatron_config[k] = ds[k]
        if overwrite_values is not None:
            megatron_config.update(overwrite_values)
        return cls.from_dict(args_dict=megatron_config)

    # ------------------------------------------------------------------ transport
    @staticmethod
    def convert_key_value_to_command_line_arg(k, v):
        if isinstance(v, bool):
            return [f"--{k}"] if v else []
        if v is None:
            return []
        return [f"--{k}", str(v)]

    def group_values(self, group: str) -> dict:
        return {n: getattr(self, n) for n, (g, _t, _d) in FIELDS.items() if g == group}

    def non_default_values(self) -> dict:
        out = {}
        for n, (_g, _t, d) in FIELDS.items():
            v = getattr(self, n)
            if v != d:
                out[n] = v
        return out

    def get_deepspeed_main_args(self):
        """argv for the launcher: runner flags that differ from their defaults, the user script,
        then ``--deepspeed_config`` and ``--megatron_config`` as base64 JSON."""
        args_list = []
        for n, (g, _t, d) in FIELDS.items():
            if g != "launcher" or n == "autotuning_run":       # the latter travels as --autotuning below
                continue
            v = getattr(self, n)
            if v != d:
                args_list.extend(self.convert_key_value_to_command_line_arg(n, v))
        if "DLTS_HOSTFILE" in os.environ and self.hostfile is None:
            args_list.extend(["--hostfile", os.environ["DLTS_HOSTFILE"]])
        if (self.autotuning_run is not None) and "--autotuning" not in args_list:
            args_list.extend(["--autotuning", self.autotuning_run])
        args_list.append(self.user_script)
        self.configure_distributed_args()
        cwd = os.getcwd()
        if self.autotuning_run is not None:
            ds_fp = os.path.join(cwd, "ds_config.json")
            with open(ds_fp, "w") as f:
                json.dump(self.deepspeed_config, f)
            args_list += ["--deepspeed_config", ds_fp]
        else:
            enc = base64.urlsafe_b64encode(json.dumps(self.deepspeed_config).encode("utf-8")).decode("utf-8")
            args_list += ["--deepspeed_config", enc]
        enc = base64.urlsafe_b64encode(json.dumps(self.non_default_values()).encode("utf-8")).decode("utf-8")
        args_list += ["--megatron_config", enc]
        return args_list

    @property
    def deepspeed_config(self) -> dict:
        """The engine-group values that are set, as the config dict the reference hands to its
        engine; ``deepspeed_extra_args`` is merged on top."""
        cfg = {k: v for k, v in self.group_values("engine").items()
               if v is not None and k not in ("deepspeed_extra_args", "deepspeed", "autotuning_run")}
        cfg.update(self.get_extra_deepspeed_args())
        return cfg

    def get_extra_deepspeed_args(self) -> dict:
        extra = copy.deepcopy(self.deepspeed_extra_args) if self.deepspeed_extra_args else {}
        return extra

    @property
    def megatron_config(self) -> dict:
        return {n: getattr(self, n) for n, (g, _t, _d) in FIELDS.items() if g not in ("engine", "launcher")}

    @property
    def all_config(self) -> dict:
        return {n: getattr(self, n) for n in FIELDS}

    def get_parent_class_value_dict_extra_ds(self):
        return self.get_extra_deepspeed_args()

    # ------------------------------------------------------------------ mutation
    def update_value(self, key: str, value):
        if key not in FIELDS:
            raise ValueError(f"{self.__class__.__name__}.update_value() to be updated property {key} "
                             "does not exist")
        setattr(self, key, value)

    def update_values(self, d: dict):
        for k, v in d.items():
            self.update_value(k, v)

    # ------------------------------------------------------------------ runtime helpers
    @property
    def params_dtype(self):
        import torch
        if self.precision == "fp16":
            return torch.half
        if self.precision == "bfloat16":
            return torch.bfloat16
        return torch.float

    def configure_distributed_args(self):
        """rank / local_rank / world_size from the environment (MPI and Slurm variable names are
        translated, megatron/neox_arguments/arguments.py:791-824)."""
        env = os.environ
        if self.deepspeed_mpi:
            env.setdefault("LOCAL_RANK", env.get("OMPI_COMM_WORLD_LOCAL_RANK", "0"))
            env.setdefault("RANK", env.get("OMPI_COMM_WORLD_RANK", "0"))
            env.setdefault("WORLD_SIZE", env.get("OMPI_COMM_WORLD_SIZE", "1"))
        if self.deepspeed_slurm:
            env["LOCAL_RANK"] = env.get("SLURM_LOCALID", "0")
            env["RANK"] = env.get("SLURM_PROCID", "0")
            env["WORLD_SIZE"] = env.get("SLURM_NTASKS", "1")
        self.update_value("local_rank", int(env.get("LOCAL_RANK", "0")))
        self.update_value("rank", int(env.get("RANK", "0")))
        self.update_value("world_size", int(env.get("WORLD_SIZE", "1")))
        if self.rank == 0:
            print(f"{self.__class__.__name__}.configure_distributed_args() using world size: "
                  f"{self.world_size} and model-parallel size: {self.model_parallel_size}", flush=True)

    def build_tokenizer(self):
        from ..tokenizer import build_tokenizer
        self.tokenizer = build_tokenizer(self)

    def initialize_tensorboard_writer(self):
        self.tensorboard_writer = None
        if self.tensorboard_dir and self.rank in (0, None):
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tensorboard_writer = SummaryWriter(log_dir=self.tensorboard_dir)
            except Exception:
                print("WARNING: TensorBoard writing requested but is not available, no TensorBoard logs "
                      "will be written.", flush=True)

    def initialize_comet(self):
        self.comet_experiment = None
        if self.use_comet and self.rank in (0, None):
            try:
                import comet_ml
                self.comet_experiment = comet_ml.Experiment(workspace=self.comet_workspace,
                                                            project_name=self.comet_project)
                self.comet_experiment.__internal_api__log_parameters__(
                    self.non_default_values(), framework="gpt-neox", source="manual", flatten_nested=True)
                if self.comet_experiment_name:
                    self.comet_experiment.set_name(self.comet_experiment_name)
                if self.comet_tags:
                    self.comet_experiment.add_tags(self.comet_tags)
                if self.comet_others:
                    self.comet_experiment.log_others(self.comet_others)
            except Exception as e:
                print(f"WARNING: Comet logging requested but unavailable ({e})", flush=True)

    def enable_logging(self):
        """Copy stdout / stderr of this process into ``log_dir/<hostname>_std{out,err}.txt``."""
        from ..obs.logging import enable_logging
        enable_logging(self)

    def print(self):
        """Dump the arguments sorted by name, defaults marked."""
        print("-------------------- arguments --------------------", flush=True)
        lines = []
        for n in sorted(FIELDS):
            v = getattr(self, n)
            d = FIELDS[n][2]
            dots = "." * max(32 - len(n), 1)
            lines.append(f"  {n} {dots} {v}" + ("" if v == d else "    (updated)"))
        for ln in sorted(lines, key=lambda x: x.lower()):
            print(ln, flush=True)
        print("---------------- end of arguments ----------------", flush=True)

    def save_yml(self, path):
        with open(path, "w") as f:
            yaml.safe_dump(json.loads(json.dumps(self.non_default_values(), default=str)), f)

    # ------------------------------------------------------------------ derivation
    @staticmethod
    def calculate_batch_parameters(dp_world_size, train_batch=None, micro_batch=None, grad_acc=None):
        """Any two of (train_batch, micro_batch, grad_acc) give the third:
        ``train_batch = micro_batch * grad_acc * dp_world_size``."""
        if train_batch is not None and micro_batch is not None and grad_acc is not None:
            return train_batch, micro_batch, grad_acc
        if train_batch is not None and micro_batch is not None:
            grad_acc = (train_batch // micro_batch) // dp_world_size
        elif train_batch is not None and grad_acc is not None:
            micro_batch = (train_batch // dp_world_size) // grad_acc
        elif micro_batch is not None and grad_acc is not None:
            train_batch = micro_batch * grad_acc * dp_world_size
        elif train_batch is not None:
            grad_acc = 1
            micro_batch = train_batch // dp_world_size
        elif micro_batch is not None:
            train_batch = micro_batch * dp_world_size
            grad_acc = 1
        else:
            raise AssertionError("Either train_batch_size or train_micro_batch_size_per_gpu needs to be provided")
        return int(train_batch), int(micro_batch), int(grad_acc)

    @staticmethod
    def check_batch_parameters(dp_world_size, train_batch, micro_batch, grad_acc):
        assert train_batch > 0, f"Train batch size: {train_batch} has to be greater than 0"
        assert micro_batch > 0, f"Micro batch size per gpu: {micro_batch} has to be greater than 0"
        assert grad_acc > 0, f"Gradient accumulation steps: {grad_acc} has to be greater than 0"
        assert train_batch == micro_batch * grad_acc * dp_world_size, (
            "Check batch related parameters. train_batch_size is not equal to micro_batch_per_gpu * "
            f"gradient_acc_step * world_size \n{train_batch} != {micro_batch} * {grad_acc} * {dp_world_size}")

    def _count_gpus(self) -> int:
        if self.hostfile is not None or os.path.exists(DEFAULT_HOSTFILE):
            pool = _parse_hostfile(self.hostfile or DEFAULT_HOSTFILE, self.include or "", self.exclude or "")
            if self.num_nodes is not None and self.num_nodes > 0:
                pool = {k: pool[k] for k in list(pool)[: self.num_nodes]}
            n = sum(len(v) for v in pool.values())
            if self.num_gpus is not None and self.num_gpus > 0:
                n = self.num_gpus * len(pool)
            return n
        if "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1:
            return int(os.environ["WORLD_SIZE"])
        import torch
        return max(torch.cuda.device_count(), 1)

    def calculate_derived(self):
        """Derive world / data-parallel size, the batch triple, precision dicts, ZeRO mirrors,
        optimizer type and lr, attention types, GQA checks, data weights, text-gen type."""
        if self.global_num_gpus is None:
            self.update_value("global_num_gpus", self._count_gpus())
        pp_size = self.pipe_parallel_size if self.pipe_parallel_size >= 1 else 1
        mp_size = self.model_parallel_size if self.model_parallel_size >= 1 else 1
        self.update_value("model_parallel_size", mp_size)
        dp_world_size = (self.global_num_gpus / pp_size) / mp_size
        if dp_world_size % 1 != 0:
            raise AssertionError(f"(global_num_gpus / pp_size) / mp_size [({self.global_num_gpus} / {pp_size}) / "
                                 f"{mp_size}] must be a whole number")
        dp_world_size = int(dp_world_size)
        if self.elasticity and self.elasticity.get("enabled"):
            # one global batch for every allowed GPU count; micro-batch and accumulation follow from this one
            from ..elasticity import compute_elastic_config
            given = [k for k in ("train_batch_size", "train_micro_batch_size_per_gpu") if getattr(self, k) is not None]
            if given and not self.elasticity.get("ignore_non_elastic_batch_info", False):
                raise AssertionError(f"elasticity is enabled: remove {given} or set ignore_non_elastic_batch_info")
            block = dict(self.elasticity, model_parallel_size=1)
            tb_e, _valid, mb_e = compute_elastic_config(block, dp_world_size)
            self.update_values({"train_batch_size": tb_e, "train_micro_batch_size_per_gpu": mb_e,
                                "gradient_accumulation_steps": tb_e // (mb_e * dp_world_size)})
        tb, mb, ga = self.calculate_batch_parameters(dp_world_size, self.train_batch_size,
                                                     self.train_micro_batch_size_per_gpu,
                                                     self.gradient_accumulation_steps)
        self.check_batch_parameters(dp_world_size, tb, mb, ga)
        self.update_values({"train_batch_size": tb, "train_micro_batch_size_per_gpu": mb,
                            "gradient_accumulation_steps": ga, "batch_size": mb,
                            "clip_grad": self.gradient_clipping})
        # precision
        if self.fp16 and self.fp16.get("enabled", False):
            if self.precision is None:
                self.update_value("precision", "fp16")
            else:
                assert self.precision == "fp16", "DeepSpeed fp16 field was set but precision conflicts"
        if self.bf16 and self.bf16.get("enabled", False):
            if self.precision is None:
                self.update_value("precision", "bfloat16")
            else:
                assert self.precision == "bfloat16", "DeepSpeed bf16 field was set but precision conflicts"
        if self.precision == "fp16":
            fp16_args = copy.deepcopy(self.fp16) if isinstance(self.fp16, dict) and self.fp16 else {"type": "fp16"}
            fp16_args["enabled"] = True
            self.update_value("fp16", fp16_args)
        elif self.precision == "bfloat16":
            if not self.bf16:
                extra = copy.deepcopy(self.deepspeed_extra_args) if self.deepspeed_extra_args else {}
                extra.update({"bf16": {"enabled": True}})
                self.update_value("deepspeed_extra_args", extra)
        else:
            self.update_value("precision", "fp32")
        # ZeRO
        if self.zero_optimization is None:
            self.zero_optimization = copy.deepcopy(ZERO_DEFAULTS)
        stage = self.zero_optimization["stage"]
        if stage in (0, 1, 2, 3):
            z = self.zero_optimization
            self.update_values({
                "zero_stage": z.get("stage", ZERO_DEFAULTS["stage"]),
                "zero_reduce_scatter": z.get("reduce_scatter", ZERO_DEFAULTS["reduce_scatter"]),
                "zero_contiguous_gradients": z.get("contiguous_gradients", ZERO_DEFAULTS["contiguous_gradients"]),
                "zero_reduce_bucket_size": z.get("reduce_bucket_size", ZERO_DEFAULTS["reduce_bucket_size"]),
                "zero_allgather_bucket_size": z.get("allgather_bucket_size", ZERO_DEFAULTS["allgather_bucket_size"]),
            })
        else:
            assert self.autotuning is not None, \
                f"Zero Stage must be an integer unless you are doing autotuning, not {stage}"
        # optimizer
        opt = self.optimizer or {"type": OPT_DEFAULT, "params": OPT_PARAMS_DEFAULTS}
        self.update_values({"optimizer_type": opt.get("type", OPT_DEFAULT),
                            "lr": opt["params"].get("lr", OPT_PARAMS_DEFAULTS["lr"])})
        if self.optimizer_type.lower() == "onebitadam":
            assert self.train_iters is not None, "OneBitAdam requires train_iters to be specified"
            self.scheduler = {"type": "WarmupDecayLR",
                              "params": {"warmup_min_lr": 0, "warmup_max_lr": self.lr,
                                         "warmup_num_steps": int(self.train_iters * self.warmup),
                                         "total_num_steps": self.lr_decay_iters or self.train_iters}}
        self.update_value("dynamic_loss_scale", self.loss_scale is None)
        self.update_value("is_pipe_parallel", self.pipe_parallel_size >= 1)
        if self.moe_num_experts > 1:
            assert self.zero_optimization["stage"] < 2, "MoE is not compatible with zero stages 2 and 3"
        # attention types
        if self.num_layers is not None:
            if self.attention_config is None:
                self.update_value("attention_config", [[["global"], self.num_layers]])
            self.update_value("attention_config", expand_attention_types(self.attention_config, self.num_layers))
            assert len(self.attention_config) == self.num_layers, \
                "Length of attention config list must equal num_layers"
            for item in self.attention_config:
                assert item in ATTENTION_TYPE_CHOICES, f"Attention type {item} not recognized"
            if "gmlp" in self.attention_config or "amlp" in self.attention_config:
                assert not self.partition_activations, "GMLP Blocks are not compatible with partition activations"
            if "mamba" in self.attention_config:
                if isinstance(self.zero_stage, int):
                    assert self.zero_stage <= 2, "Zero stage 3 not compatible with Mamba"
                assert self.hidden_dropout == 0.0, "Mamba does not yet have dropout implemented"
            if "rwkv" in self.attention_config:
                assert self.model_parallel_size == 1, "RWKV not currently compatible with model parallelism"
                if isinstance(self.zero_stage, int):
                    assert self.zero_stage <= 2, "Zero stage 3 not compatible with RWKV"
                assert self.hidden_dropout == 0.0, "RWKV does not yet have dropout implemented"
        if self.sparsity_config is None:
            self.update_value("sparsity_config", {})
        # GQA / MQA
        if self.num_kv_heads is not None and self.num_attention_heads is not None:
            assert self.num_attention_heads % self.num_kv_heads == 0, \
                "num_kv_heads must evenly divide num_attention_heads and be no greater than it"
            if self.num_kv_heads < self.num_attention_heads:
                assert not self.sparsity_config, "Sparse attention not compatible with GQA or MQA"
                assert all(t in ("flash", "global") for t in (self.attention_config or [])), \
                    "GQA / MQA currently only compatible with Flash or standard global/sliding window Attention"
                assert self.num_kv_heads % self.model_parallel_size == 0, \
                    "Number of KV heads must be at least model_parallel_size for now!"
        # data weights
        for split in ("train", "valid", "test"):
            paths = getattr(self, f"{split}_data_paths") or getattr(self, f"pos_{split}_data_paths")
            if paths and getattr(self, f"{split}_data_weights") is None:
                setattr(self, f"{split}_data_weights", [1.0] * len(paths))
        if self.train_label_data_paths:
            assert self.train_data_paths and not self.data_path, \
                "Must use `train_label_data_paths` with `train_data_paths`, not `data_path`"
        if self.text_gen_type is None:
            self.update_value("text_gen_type", "input-file" if self.sample_input_file else "unconditional")

    # ------------------------------------------------------------------ validation
    @staticmethod
    def validate_keys() -> bool:
        """No field name may be declared twice across the schema groups."""
        seen = set()
        for g, entries in SCHEMA.items():
            for n, _t, _d in entries:
                if n in seen:
                    logging.error(f"NeoXArgs.validate_keys() duplicate of item: {n} (group {g})")
                    return False
                seen.add(n)
        return True

    def validate_types(self) -> bool:
        for n, (_g, t, _d) in FIELDS.items():
            v = getattr(self, n)
            if not type_ok(v, t):
                logging.error(f"{self.__class__.__name__}.validate_types() {n}: '{v}' ({type(v).__name__}) "
                              f"not of type {t}")
                return False
            if t.startswith("one_of[") and isinstance(v, str):
                setattr(self, n, _canonical_choice(t, v))
        for name in ("optimizer", "scheduler"):
            v = getattr(self, name)
            if isinstance(v, dict):
                if "type" not in v or not isinstance(v["type"], str):
                    logging.error(f"{self.__class__.__name__}.validate_types() {name}: key 'type' must be a string")
                    return False
                if "params" not in v or not isinstance(v["params"], dict):
                    logging.error(f"{self.__class__.__name__}.validate_types() {name}: key 'params' must be a dict")
                    return False
        for name in ("fp16", "amp", "flops_profiler"):
            v = getattr(self, name)
            if isinstance(v, dict):
                if "enabled" not in v or not isinstance(v["enabled"], bool):
                    logging.error(f"{self.__class__.__name__}.validate_types() {name}: must contain key 'enabled' "
                                  "of type bool")
                    return False
        return True

    def validate_values(self) -> bool:
        err = lambda msg: (logging.error(f"{self.__class__.__name__}.validate_values() {msg}"), False)[1]
        if not self.deepspeed:
            return err("Deepspeed is not set to True; the engine of this framework takes the same switch.")
        if self.lr is None:
            return err("lr is None")
        for req in ("num_layers", "hidden_size", "num_attention_heads", "max_position_embeddings", "seq_length"):
            if getattr(self, req) is None:
                return err(f"{req} is None")
        if self.hidden_size % self.num_attention_heads != 0 and "mamba" not in self.attention_config:
            return err("hidden_size must be divisible by num_attention_heads")
        if self.seq_length is not None and self.max_position_embeddings < self.seq_length:
            return err("max_position_embeddings must be bigger or equal seq_length")
        if self.min_lr is not None and self.min_lr > self.lr:
            return err("min_lr must be smaller or equal lr")
        if self.save is not None and self.checkpoint_factor is None and self.extra_save_iters is None:
            return err("checkpoint_factor or extra_save_iters must be defined if save is defined")
        if self.checkpoint_activations and self.checkpoint_num_layers is not None:
            if self.num_layers % self.checkpoint_num_layers != 0:
                return err("num_layers must be divisible by checkpoint_num_layers")
        if self.fp16_lm_cross_entropy and self.precision != "fp16":
            return err("lm cross entropy in fp16 only support in fp16 mode.")
        paths = [self.train_data_paths, self.valid_data_paths, self.test_data_paths]
        if any(p is not None for p in paths) and not all(p is not None for p in paths):
            return err("One of train/valid/test data_path(s) is given, but not all")
        if self.train_data_paths is not None and self.data_path is not None:
            return err("data_path and train/valid/test data_paths are mutually exclusive")
        for split in ("train", "valid", "test"):
            p, w = getattr(self, f"{split}_data_paths"), getattr(self, f"{split}_data_weights")
            if p is not None and w is not None and len(p) != len(w):
                return err(f"{split}_data_weights must have the same length as {split}_data_paths")
        if self.num_unique_layers is not None:
            if self.num_unique_layers > self.num_layers:
                return err("number of unique layers must be smaller than or equal num_layers")
            if self.num_layers % self.num_unique_layers != 0:
                return err("number of layers must be divisible by number of unique layers")
        if self.sequence_parallel and self.model_parallel_size > 1:
            if self.seq_length % self.model_parallel_size != 0:
                return err("seq_length must be divisible by model_parallel_size under sequence parallelism")
        if self.moe_num_experts > 1:
            ep = max(self.moe_expert_parallel_size, 1)
            if self.moe_num_experts % ep != 0:
                return err("moe_num_experts must be divisible by moe_expert_parallel_size")
        return True


def _canonical_choice(t: str, v: str) -> str:
    """Literal values are matched case-insensitively and stored in the schema's spelling."""
    for c in _split_top(t[len("one_of["):-1]):
        c = c.strip().strip("'\"")
        if c.lower() == v.lower():
            return c
    return v


def gen_docs() -> str:
    """Markdown listing of every argument by group (the counterpart of configs/gen_docs.py)."""
    out = ["# NeoX arguments", ""]
    for g, entries in SCHEMA.items():
        out.append(f"## {g}")
        out.append("")
        out.append("| name | type | default |")
        out.append("|---|---|---|")
        for n, t, d in entries:
            out.append(f"| `{n}` | `{t}` | `{d!r}` |")
        out.append("")
    return "\n".join(out)
