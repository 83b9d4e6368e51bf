"""Import-compatibility package: ``megatron.<module>`` resolves to the module of ``gpt_neox_b200`` that
provides the same API, so code written against the reference's package layout (``from megatron.neox_arguments
import NeoXArgs``, ``from megatron import mpu``, ``from megatron.training import pretrain`` ...) runs unchanged.

Aliases are resolved lazily by a meta-path finder; ``megatron.model.transformer`` maps to
``gpt_neox_b200.models.transformer`` and so on for every submodule under an aliased package.
"""
import importlib
import importlib.abc
import importlib.util
import sys

_PREFIXES = [
    ("megatron.model.rwkv.v6.rwkv", "gpt_neox_b200.models.rwkv"),
    ("megatron.model.rwkv.v6", "gpt_neox_b200.models.rwkv"),
    ("megatron.model.mamba.mamba", "gpt_neox_b200.models.mamba"),
    ("megatron.mup_substitute", "gpt_neox_b200.mup"),
    ("megatron.devutil", "gpt_neox_b200.utils.devutil"),
    ("megatron.neox_arguments.arguments", "gpt_neox_b200.config.arguments"),
    ("megatron.neox_arguments", "gpt_neox_b200.config"),
    ("megatron.mpu", "gpt_neox_b200.parallel"),
    ("megatron.model", "gpt_neox_b200.models"),
    ("megatron.data", "gpt_neox_b200.data"),
    ("megatron.tokenizer", "gpt_neox_b200.tokenizer"),
    ("megatron.utils", "gpt_neox_b200.utils.common"),
    ("megatron.training", "gpt_neox_b200.training"),
    ("megatron.initialize", "gpt_neox_b200.initialize"),
    ("megatron.checkpointing", "gpt_neox_b200.ckpt.checkpointing"),
    ("megatron.learning_rates", "gpt_neox_b200.engine.lr"),
    ("megatron.optimizers", "gpt_neox_b200.optimizers"),
    ("megatron.logging", "gpt_neox_b200.obs.logging"),
    ("megatron.text_generation_utils", "gpt_neox_b200.text_generation_utils"),
    ("megatron.gradient_noise_scale", "gpt_neox_b200.gradient_noise_scale"),
    ("megatron.fused_kernels", "gpt_neox_b200.ops.softmax"),
]


_NESTED = ("gpt_neox_b200.models.rwkv", "gpt_neox_b200.models.mamba")


def _target(name):
    for src, dst in _PREFIXES:
        if name == src:
            return dst
        if name.startswith(src + "."):
            return dst + name[len(src):]
    return None


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self.target = target

    def create_module(self, spec):
        real = importlib.import_module(self.target)
        self.real_spec = real.__spec__
        return real

    def exec_module(self, module):
        # the import machinery has just stamped the alias spec onto the real module: put its own spec back, so
        # that relative imports inside it keep resolving against its real package
        module.__spec__ = self.real_spec
        if self.target in _NESTED and not hasattr(module, "__path__"):
            module.__path__ = []          # a plain module here, a package in the reference: let submodule aliases resolve


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        t = _target(fullname)
        if t is None:
            return None
        try:
            if importlib.util.find_spec(t) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.util.spec_from_loader(fullname, _AliasLoader(t))


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name):
    t = _target(f"megatron.{name}")
    if t is None:
        raise AttributeError(name)
    return importlib.import_module(f"megatron.{name}")


def print_rank_0(*message):
    from gpt_neox_b200.utils.common import print_rank_0 as _p
    _p(*message)
