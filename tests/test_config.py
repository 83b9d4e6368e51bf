"""Config system: constructors, CLI round trip deepy -> per-rank args, derived values, usage lint
(reference: tests/neox_args/*, tests/unit/test_arguments.py)."""
import os
import re

import pytest
import yaml

from common import ROOT, tiny_config
from gpt_neox_b200.config import NeoXArgs
from gpt_neox_b200.config.arguments import FIELDS


def test_from_dict_derives_batch_sizes_and_precision():
    a = NeoXArgs.from_dict(tiny_config(global_num_gpus=4, train_micro_batch_size_per_gpu=2,
                                       gradient_accumulation_steps=3, precision="bfloat16"))
    assert a.train_batch_size == 2 * 3 * 4
    import torch
    assert a.params_dtype == torch.bfloat16
    assert a.attention_config == ["global", "global"]
    with pytest.raises(Exception):
        NeoXArgs.from_dict(tiny_config(hidden_size=65))                    # not divisible by heads
    with pytest.raises(TypeError):
        NeoXArgs.from_dict(tiny_config(no_such_argument=1))


def test_duplicate_keys_across_yaml_files_are_rejected(tmp_path):
    cfg = tiny_config()
    (tmp_path / "a.yml").write_text(yaml.safe_dump(cfg))
    (tmp_path / "b.yml").write_text(yaml.safe_dump({"hidden_size": 128}))
    with pytest.raises(ValueError, match="duplicate"):
        NeoXArgs.from_ymls([str(tmp_path / "a.yml"), str(tmp_path / "b.yml")])


def test_cli_round_trip_deepy_to_rank_args(tmp_path):
    cfg = tiny_config(num_layers=3, hidden_size=96, num_attention_heads=3)
    (tmp_path / "model.yml").write_text(yaml.safe_dump(cfg))
    (tmp_path / "setup.yml").write_text(yaml.safe_dump({"log_dir": str(tmp_path / "logs"), "master_port": 29999}))
    for argv in (["train.py", "-d", str(tmp_path), "model", "setup.yml"],
                 ["train.py", str(tmp_path / "model.yml"), str(tmp_path / "setup.yml")]):
        a = NeoXArgs.consume_deepy_args(argv)
        assert a.user_script == "train.py" and a.num_layers == 3 and a.master_port == 29999
        main_args = a.get_deepspeed_main_args()
        assert "--master_port" in main_args and main_args[main_args.index("--master_port") + 1] == "29999"
        i = main_args.index("train.py")
        b = NeoXArgs.consume_neox_args(input_args=main_args[i + 1:])
        for k in ("num_layers", "hidden_size", "num_attention_heads", "seq_length", "optimizer", "train_batch_size",
                  "zero_optimization"):
            assert getattr(a, k) == getattr(b, k), k


def test_every_neox_args_attribute_used_in_the_package_is_declared():
    pat = re.compile(r"neox_args\.([A-Za-z_][A-Za-z0-9_]*)")
    methods = {n for n in dir(NeoXArgs)}
    dynamic = {"tokenizer", "padded_vocab_size", "params_dtype", "tensorboard_writer", "comet_experiment",
               "iteration", "do_train", "do_valid", "do_test", "curriculum_seqlen", "is_pipe_parallel",
               "dim_att", "head_size", "ffn_dim", "global_num_gpus", "rank", "local_rank", "world_size",
               "py"}                       # "neox_args.py" in citations of the reference file name
    unknown = {}
    for root, _, files in os.walk(os.path.join(ROOT, "gpt_neox_b200")):
        for f in files:
            if f.endswith(".py"):
                for name in pat.findall(open(os.path.join(root, f)).read()):
                    if name not in FIELDS and name not in methods and name not in dynamic:
                        unknown.setdefault(name, f)
    assert not unknown, unknown


def test_no_field_is_declared_twice():
    from gpt_neox_b200.config.schema import SCHEMA
    seen = {}
    for group, rows in SCHEMA.items():
        for name, _t, _d in rows:
            assert name not in seen, f"{name} in {group} and {seen[name]}"
            seen[name] = group


def test_elasticity_keeps_one_global_batch_over_gpu_counts():
    import pytest
    from common import tiny_config
    from gpt_neox_b200.elasticity import ElasticityError, compute_elastic_config, valid_gpu_counts
    block = {"enabled": True, "max_train_batch_size": 2000, "micro_batch_sizes": [2, 4, 6], "min_gpus": 1,
             "max_gpus": 64, "prefer_larger_batch": True}
    batch, valid, _ = compute_elastic_config(block)
    assert batch <= 2000 and valid == valid_gpu_counts(batch, [2, 4, 6], 1, 64)
    assert len(valid) >= 20 and {1, 2, 4, 8, 24}.issubset(valid)
    for g in valid:                                                   # every valid size really forms the batch
        assert any(batch % (m * g) == 0 for m in (2, 4, 6))
    seen = set()
    for world in (8, 12, 24):
        cfg = tiny_config(elasticity=block, global_num_gpus=world)
        for k in ("train_micro_batch_size_per_gpu", "gradient_accumulation_steps"):
            cfg.pop(k)
        a = NeoXArgs.from_dict(cfg)
        assert a.train_batch_size == batch
        assert a.train_micro_batch_size_per_gpu * a.gradient_accumulation_steps * world == batch
        seen.add(a.train_micro_batch_size_per_gpu)
    assert seen <= {2, 4, 6}
    with pytest.raises(ElasticityError):
        compute_elastic_config(block, 7 * 11)                         # 77 ranks cannot divide the batch
    with pytest.raises(AssertionError):
        NeoXArgs.from_dict(tiny_config(elasticity=block, global_num_gpus=8))   # explicit batch keys conflict
    small, v2, _ = compute_elastic_config(dict(block, prefer_larger_batch=False))
    assert len(v2) == len(valid) and small <= batch


def test_argument_reference_document_is_current():
    """configs/neox_arguments.md is generated from the schema; a schema change must regenerate it."""
    import importlib.util
    import os
    from common import ROOT
    spec = importlib.util.spec_from_file_location("gen_docs_script", os.path.join(ROOT, "configs", "gen_docs.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.main(["--check"]) == 0
