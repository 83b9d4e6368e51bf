"""Engine-side observability switches: wall_clock_breakdown, flops_profiler, comms_logger, dump_state
(declared in the reference at megatron/neox_arguments/deepspeed_args.py:146-173,238)."""
import io

import torch

from common import run_distributed, tiny_config


def _train(rank, world, cfg, steps=4):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world, train_iters=steps, lr_decay_iters=steps))
    a.configure_distributed_args()
    a.build_tokenizer()
    import contextlib
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        model = training.pretrain(a)
    out = dict(stdout=buf.getvalue(), timer_values=model.timer_values)
    if model.flops_profiler is not None:
        out["flops"] = model.flops_profiler.totals().get("", 0.0)
        out["stats"] = {n: (s["calls"], s["cls"]) for n, s in model.flops_profiler.stats.items() if s["calls"]}
    if model.comms_logger is not None:
        out["comm_ops"] = {op: {b: r[0] for b, r in d.items()} for op, d in model.comms_logger.records.items()}
        import torch.distributed as dist
        out["restored"] = not hasattr(dist.all_reduce, "neox_comms_wrapper")
    return out


def test_wall_clock_breakdown_and_dump_state():
    cfg = tiny_config(use_cpu_initialization=True, wall_clock_breakdown=True, steps_per_print=2, dump_state=True,
                      gradient_accumulation_steps=2)
    r = run_distributed(_train, 1, cfg)[0]
    lines = [l for l in r["stdout"].splitlines() if l.startswith("time (ms) per step")]
    assert len(lines) == 2                                            # 4 steps, printed every 2
    for phase in ("forward", "backward", "grad_reduce", "optimizer", "param_gather"):
        assert phase + ":" in lines[0] and r["timer_values"][phase] >= 0
    assert r["timer_values"]["forward"] > 0 and r["timer_values"]["backward"] > 0
    assert "engine state:" in r["stdout"] and "zero_stage" in r["stdout"]


def test_wall_clock_breakdown_under_pipeline_parallelism():
    cfg = tiny_config(use_cpu_initialization=True, wall_clock_breakdown=True, steps_per_print=2, pipe_parallel_size=2,
                      gradient_accumulation_steps=2)
    r = run_distributed(_train, 2, cfg)
    for rr in r:
        assert rr["timer_values"]["pipe_comm"] > 0 and rr["timer_values"]["forward"] > 0


def test_flops_profiler_counts_the_matmuls(tmp_path):
    out_file = str(tmp_path / "flops.txt")
    cfg = tiny_config(use_cpu_initialization=True, make_vocab_size_divisible_by=64,
                      flops_profiler={"enabled": True, "profile_step": 2, "module_depth": -1, "top_modules": 2,
                                      "detailed": True, "output_file": out_file})
    r = run_distributed(_train, 1, cfg, 3)[0]
    h, L, s, b = 64, 2, 32, 2
    vocab = 128                                                       # 100 synthetic ids padded to a multiple of 64
    tokens = s * b
    expect = L * (2 * tokens * 12 * h * h + 4 * b * s * s * h) + 2 * tokens * h * vocab
    assert abs(r["flops"] - expect) / expect < 1e-6, (r["flops"], expect)
    text = open(out_file).read()
    assert "forward FLOPs on this rank" in text and "depth 2:" in text and "top flops" in text
    assert any(cls == "ParallelSelfAttention" for _, cls in r["stats"].values())
    assert all(calls == 1 for calls, _ in r["stats"].values())        # one profiled step, one micro-batch


def test_comms_logger_tabulates_collectives():
    cfg = tiny_config(use_cpu_initialization=True, comms_logger={"enabled": True, "verbose": False, "prof_all": True,
                                                                 "debug": False})
    r = run_distributed(_train, 2, cfg, 2)[0]
    assert "all_reduce" in r["comm_ops"] and sum(r["comm_ops"]["all_reduce"].values()) >= 2
    assert "comm. op" in r["stdout"] and "busbw (GB/s)" in r["stdout"]
    assert r["restored"]


def test_comms_logger_prof_ops_filter_and_bus_factor():
    from gpt_neox_b200.obs.profiling import CommsLogger, _bus_factor
    assert _bus_factor("all_reduce", 8) == 2 * 7 / 8 and _bus_factor("all_gather_into_tensor", 4) == 3 / 4
    assert _bus_factor("broadcast", 8) == 1.0 and _bus_factor("all_reduce[nvlink]", 2) == 1.0
    c = CommsLogger(prof_all=False, prof_ops=["all_reduce"])
    with c.observe("all_reduce", 1024, 4):
        pass
    with c.observe("broadcast", 64, 4):
        pass
    assert list(c.records) == ["all_reduce"] and c.records["all_reduce"][1024][0] == 1
    assert "1.00 KB" in c.summary()


def _train_csv(rank, world, cfg):
    _train(rank, world, cfg, 4)
    return True


def test_csv_monitor_writes_one_file_per_scalar(tmp_path):
    cfg = tiny_config(use_cpu_initialization=True, log_interval=1,
                      csv_monitor={"enabled": True, "output_path": str(tmp_path), "job_name": "job"})
    run_distributed(_train_csv, 1, cfg)
    rows = (tmp_path / "job" / "train_lm_loss.csv").read_text().strip().splitlines()
    assert rows[0] == "step,train_lm_loss" and len(rows) == 5
    assert [int(r.split(",")[0]) for r in rows[1:]] == [1, 2, 3, 4]
    assert (tmp_path / "job" / "train_learning_rate.csv").exists()
