"""Every shipped model config loads through NeoXArgs (reference: tests/neox_args/test_neoxargs_load.py)."""
import contextlib
import glob
import io
import os

import pytest
import yaml

from common import ROOT
from gpt_neox_b200.config import NeoXArgs

CONF = os.path.join(ROOT, "configs")
SETUP_ONLY = ("local_setup", "slurm_local", "text_generation", "cpu_mock_config", "prof.yml")
OVERLAYS = ("sparse.yml", "llama/train_config.yml")                        # no model shape of its own: applied on top of a model config
FILES = sorted(os.path.relpath(f, CONF) for ext in ("*.yml", "autotuning_configs/*.json")
               for f in glob.glob(os.path.join(CONF, "**", ext), recursive=True))
MODELS = [f for f in FILES if not any(s in f for s in SETUP_ONLY)]


@pytest.mark.parametrize("rel", MODELS)
def test_model_config_loads(rel):
    paths = [os.path.join(CONF, rel)]
    with open(paths[0]) as f:
        keys = set(yaml.safe_load(f))
    with open(os.path.join(CONF, "local_setup.yml")) as f:
        setup_keys = set(yaml.safe_load(f))
    if not (keys & setup_keys) and not rel.startswith("bench"):
        paths.append(os.path.join(CONF, "local_setup.yml"))
    over = {"global_num_gpus": 8}
    if rel in OVERLAYS:
        paths.insert(0, os.path.join(CONF, "llama", "7B.yml") if rel.startswith("llama")
                     else os.path.join(CONF, "125M.yml"))
        keys |= {"train_micro_batch_size_per_gpu", "checkpoint_factor"}
    if not keys & {"train_micro_batch_size_per_gpu", "train_batch_size"}:
        over["train_micro_batch_size_per_gpu"] = 1          # shape-only files (llama/*) are combined with a train config
    if not keys & {"checkpoint_factor", "extra_save_iters"}:
        over["checkpoint_factor"] = 1000
    with contextlib.redirect_stdout(io.StringIO()):
        a = NeoXArgs.from_ymls(paths, overwrite_values=over)
    assert a.num_layers > 0
    if not any(t in ("mamba", "rwkv") for t in a.attention_config):
        assert a.hidden_size % a.num_attention_heads == 0
    assert a.train_batch_size == a.train_micro_batch_size_per_gpu * a.gradient_accumulation_steps * \
        (8 // (a.model_parallel_size * max(1, a.pipe_parallel_size)))
    assert a.precision in ("bfloat16", "fp16", "fp32")


@pytest.mark.parametrize("rel", [f for f in FILES if any(s in f for s in SETUP_ONLY)])
def test_setup_files_are_valid_yaml_with_known_keys(rel):
    from gpt_neox_b200.config.arguments import FIELDS
    with open(os.path.join(CONF, rel)) as f:
        d = yaml.safe_load(f)
    unknown = [k for k in d if k.replace("-", "_") not in FIELDS]
    assert not unknown, unknown
