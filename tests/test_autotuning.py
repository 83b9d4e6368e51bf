"""Autotuner: memory model, search space, tuner logic with a fake experiment runner, the training-side
profile window, and one end-to-end ``deepy.py --autotuning tune`` on CPU (reference surface:
megatron/neox_arguments/arguments.py:95-101,497-505, configs/autotuning_configs/*.json)."""
import json
import os
import sys

import pytest

from common import ROOT, free_port, tiny_config
from gpt_neox_b200 import autotuning as at

NEOX = {"hidden-size": 4096, "num-layers": 32, "num-attention-heads": 32, "seq-length": 2048,
        "no-weight-tying": True, "vocab_size": 50432, "checkpoint-activations": True}


def test_memory_model_orders_stages_and_batches():
    info = at.model_info(NEOX)
    assert 6.0e9 < info["params"] < 7.5e9
    m0, m1, m2 = (at.memory_per_gpu(info, s, 4, dp=8) for s in (0, 1, 2))
    assert m0 > m1 > m2
    assert at.memory_per_gpu(info, 1, 8, dp=8) > m1
    assert at.memory_per_gpu(info, 1, 4, dp=1) == pytest.approx(at.memory_per_gpu(info, 0, 4, dp=1))
    top = at.max_micro_batch(info, 1, 8, 0.9 * 180e9, 1024)
    assert top >= 4 and at.memory_per_gpu(info, 1, top, 8) <= 0.9 * 180e9 < at.memory_per_gpu(info, 1, 2 * top, 8)
    assert at.max_micro_batch(info, 0, 1, 10e9, 1024) == 0          # 6.9B parameters do not fit 10 GB at all


def test_search_space_from_stage_list():
    ds = {"zero_optimization": {"stage": [0, 1, 2, 3], "reduce_bucket_size": 5e8},
          "autotuning": {"enabled": True, "num_tuning_micro_batch_sizes": 3, "max_train_batch_size": 1024}}
    exps = at.build_space(ds, at.model_info(NEOX), world_size=8)
    stages = sorted({e["zero_optimization"]["stage"] for e in exps})
    assert stages == [0, 1, 2]                                       # stage 3 is not offered
    for e in exps:
        assert e["train_batch_size"] == e["train_micro_batch_size_per_gpu"] * e["gradient_accumulation_steps"] * 8
        assert e["train_batch_size"] <= 1024 and e["zero_optimization"]["reduce_bucket_size"] == 5e8
    per_stage = [e["train_micro_batch_size_per_gpu"] for e in exps if e["zero_optimization"]["stage"] == 1]
    assert per_stage == sorted(per_stage) and len(per_stage) == 3


@pytest.mark.parametrize("tuner", ["gridsearch", "random", "model_based"])
def test_tuner_picks_best_and_prunes_after_failure(tmp_path, tuner):
    ds = {"zero_optimization": {"stage": [0, 1]}, "train_micro_batch_size_per_gpu": 1,
          "autotuning": {"enabled": True, "tuner_type": tuner, "num_tuning_micro_batch_sizes": 4,
                         "results_dir": str(tmp_path / "res"), "exps_dir": str(tmp_path / "exps"),
                         "tuner_early_stopping": 10}}
    ran = []

    def runner(exp, exp_dir):
        s, b = exp["zero_optimization"]["stage"], exp["train_micro_batch_size_per_gpu"]
        ran.append((s, b))
        info = at.model_info(NEOX)
        top = at.max_micro_batch(info, s, 8, 0.9 * 180e9, 1024)
        if s == 0 and b >= top // 2:
            return None                                              # stage 0 "runs out of memory" early
        return {"throughput": b * (1.0 if s == 1 else 0.9) / (1 + 0.01 * b), "latency": 1.0 / b, "flops": 1.0}

    t = at.Autotuner(ds, NEOX, 8, runner, log=lambda *_: None)
    best = t.tune()
    top1 = at.max_micro_batch(at.model_info(NEOX), 1, 8, 0.9 * 180e9, 1024)
    assert best["zero_optimization"]["stage"] == 1 and best["train_micro_batch_size_per_gpu"] == top1
    statuses = {r["name"]: r["status"] for r in t.records}
    assert "failed" in statuses.values()
    if tuner != "random":                                            # in rising order the larger sizes are never run
        assert "pruned" in statuses.values()
        failed = [r for r in t.records if r["status"] == "failed"]
        assert len(failed) == 1
    opt = json.load(open(tmp_path / "res" / "ds_config_optimal.json"))
    assert opt["zero_optimization"]["stage"] == 1 and "autotuning" not in opt
    assert opt["train_batch_size"] == top1 * 8
    assert "best: " + best["name"] in open(tmp_path / "res" / "summary.txt").read()


def test_latency_metric_minimises(tmp_path):
    ds = {"zero_optimization": {"stage": 1}, "autotuning": {"enabled": True, "metric": "latency",
          "results_dir": str(tmp_path / "r"), "exps_dir": str(tmp_path / "e")}}
    t = at.Autotuner(ds, NEOX, 8, lambda e, d: {"latency": e["train_micro_batch_size_per_gpu"], "throughput": 1, "flops": 1},
                     log=lambda *_: None)
    best = t.tune()
    assert best["train_micro_batch_size_per_gpu"] == min(r["train_micro_batch_size_per_gpu"] for r in t.records)
    with pytest.raises(ValueError):
        at.settings({"autotuning": {"metric": "speed"}})


def test_profile_window_writes_metrics(tmp_path):
    path = str(tmp_path / "m.json")
    w = at.ProfileWindow(2, 4, path, samples_per_step=16, flops_per_step=1e12)
    assert [w.after_step(i) for i in (1, 2, 3)] == [False, False, False]
    assert w.after_step(4) is True
    m = json.load(open(path))
    assert m["throughput"] == pytest.approx(16 / m["latency"]) and m["flops"] == pytest.approx(1e12 / m["latency"])
    with pytest.raises(ValueError):
        at.ProfileWindow(3, 3, path, 1)


def test_deepy_autotuning_end_to_end_on_cpu(tmp_path, monkeypatch):
    """Two ZeRO stages x two micro-batch sizes of a tiny CPU model, each a real launch of train.py that the
    profile window ends after four steps."""
    import yaml
    cfg = tiny_config(zero_optimization={"stage": [0, 1]}, train_iters=50, use_cpu_initialization=True,
                      master_port=free_port(), train_micro_batch_size_per_gpu=1,
                      autotuning={"enabled": True, "start_profile_step": 2, "end_profile_step": 4,
                                  "num_tuning_micro_batch_sizes": 2, "max_train_micro_batch_size_per_gpu": 4,
                                  "results_dir": str(tmp_path / "res"), "exps_dir": str(tmp_path / "exps")})
    cfg.pop("global_num_gpus")
    (tmp_path / "c.yml").write_text(yaml.safe_dump(cfg))
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("PYTHONPATH", ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    sys.path.insert(0, ROOT)
    import deepy
    rc = deepy.main([os.path.join(ROOT, "train.py"), "--autotuning", "tune", str(tmp_path / "c.yml")])
    assert rc == 0
    summary = (tmp_path / "res" / "summary.txt").read_text()
    assert summary.count(" ok ") == 4 and "best: z" in summary
    opt = json.load(open(tmp_path / "res" / "ds_config_optimal.json"))
    assert opt["zero_optimization"]["stage"] in (0, 1) and opt["train_micro_batch_size_per_gpu"] in (2, 4)
    m = json.load(open(tmp_path / "exps" / "z1_mbs4_gas1" / "metrics.json"))
    assert m["throughput"] > 0
