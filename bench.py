#!/usr/bin/env python
"""Headline benchmark: bf16 training throughput (tokens/s, TFLOP/s per GPU) of the Pythia-6.9B
shape on N GPUs of one node, synthetic tokens, random-init weights.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--model pythia-6-9B] [--impl ours|reference|library]

``--impl library`` runs the same model shape, batch layout and optimizer step in plain PyTorch on
vendor kernels (cuBLAS, flash-attn, NCCL; baseline/library_arm.py) and prints the same JSON line with
``"impl": "library"``: a same-box baseline at step level.  It is not the reference implementation.
At ``--gpus 8`` the default run also measures the second headline configuration, GPT-NeoX-20B on
tp4 x pp2, in child processes and reports it under ``"neox_20b"``.

N = 1: TP 1;  N >= 2: TP 2 + sequence parallel x DP N/2, ZeRO-1.  Micro-batch 4, global batch
64 * N sequences of 2048 tokens (512 at N = 8): per-GPU work is fixed as N grows (weak scaling).
Two measurements per run, both over exactly K optimizer steps after W warm-up steps, bracketed by
barrier + synchronize, max over ranks:
  value  device-timed (CUDA events) with the batches already resident on the device;
  e2e    the same steps driven through the framework's own data loader: every micro-batch is
         copied from pinned host memory and the loss is read back to the host every step.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=("ours", "reference", "library"))
    p.add_argument("--model", type=str, default=os.environ.get("NEOX_BENCH_MODEL", "pythia-6-9B"))
    p.add_argument("--micro-batch", type=int, default=None)
    p.add_argument("--gas", type=int, default=None, help="override gradient accumulation steps")
    p.add_argument("--mode", type=str, default="fused", choices=("fused", "nccl_baseline"))
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-20b", action="store_true", help="at --gpus 8: skip the NeoX-20B (tp4 x pp2) measurement")
    p.add_argument("--json-out", type=str, default=None, help="rank 0 also writes its JSON line to this file")
    p.add_argument("--fp8", action="store_true",
                   help="run the linear layers' GEMMs (forward, dgrad, wgrad) on the fp8 tensor cores with delayed "
                        "scaling; reported under dtype 'fp8' and never as the bf16 headline")
    p.add_argument("--fp8-recipe", type=str, default="delayed", choices=("delayed", "mxfp8"),
                   help="with --fp8: per-tensor delayed scaling, or block scaling (one power-of-two scale per 32 elements)")
    p.add_argument("--kernel-table", type=str, default=None,
                   help="after the timed regions, run one more (untimed) step under torch.profiler and write the "
                        "per-kernel device-time table of rank 0 to this file")
    return p.parse_args()


def reference_arm(args):
    """The unmodified reference, if it could be installed under baseline/_ref."""
    ref = os.path.join(REPO, "baseline", "_ref")
    why = None
    if not os.path.isdir(ref):
        why = ("reference not installed: baseline/_ref is absent (the reference tree has no setup.py / pyproject.toml, "
               "so the offline pip install refuses it, and its DeepSpeed runtime is not in the wheelhouse)")
    else:
        sys.path.insert(0, ref)
        try:
            import deepspeed  # noqa: F401  (the reference's whole runtime)
        except Exception as e:
            why = f"reference needs DeepSpeed (EleutherAI DeeperSpeed fork), which is not installable offline: {type(e).__name__}"
        if why is None:
            try:
                import megatron  # noqa: F401
            except Exception as e:
                why = f"reference package does not import on this image: {type(e).__name__}: {e}"
    if why is None:
        why = "reference entry point train.py hard-requires its DeepSpeed launcher; not runnable here"
    if int(os.environ.get("RANK", "0")) == 0:          # one line per job, also when launched by torchrun
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def library_arm(args):
    """Same shape, same batch layout, same step - plain PyTorch on library kernels (baseline/library_arm.py)."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(REPO, "baseline"))
    import library_arm as la

    n = args.gpus
    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if args.model not in la.SHAPES:
        if rank == 0:
            print(json.dumps({"impl": "library", "unavailable": f"the library arm has no {args.model} layout"}))
        return 0
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if n > 1:
        dist.init_process_group("nccl", device_id=dev)
    seq = 2048
    micro = args.micro_batch or (4 if "6-9B" in args.model else 16)
    model, opt, tp, dp, dp_rank = la.build(args.model, n, rank, dev, seq)
    per_gpu_seqs = 64 if "6-9B" in args.model else 128
    gas = args.gas or (per_gpu_seqs * n) // (micro * dp)
    global_batch = micro * gas * dp
    g = torch.Generator(device="cpu")
    g.manual_seed(1234 + dp_rank)
    pool = [torch.randint(0, 50277, (micro, seq + 1), generator=g, dtype=torch.int64).to(dev) for _ in range(min(gas, 8))]
    host = [torch.randint(0, 50277, (micro, seq + 1), generator=g, dtype=torch.int64).pin_memory() for _ in range(gas)]

    def barrier_sync():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if n > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def device_step():
        return la.train_step(model, opt, [pool[i % len(pool)] for i in range(gas)])

    def e2e_step():
        loss = la.train_step(model, opt, [h.to(dev, non_blocking=True) for h in host])
        return float(loss.item())

    for _ in range(args.warmup):
        device_step()
    sampler = ClockSampler(local_rank)
    barrier_sync()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        device_step()
    e1.record()
    barrier_sync()
    clocks = sampler.stop() if rank == 0 else None
    dev_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    e2e = None
    if not args.no_e2e:
        e2e_step()
        barrier_sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            last = e2e_step()
        barrier_sync()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1000.0) / args.steps
        e2e = {"value": global_batch * seq / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": gas * micro * (seq + 1) * 8, "d2h_bytes_per_step": 4, "final_loss": last}
    if rank == 0:
        tokens = global_batch * seq
        out = {"metric": "tokens_per_sec", "value": tokens / (dev_ms / 1000.0), "unit": "tokens/s", "n_gpus": n,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True,
               "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic tokens, random-init weights",
               "tflops_per_gpu": la.flops_per_step(args.model, global_batch, seq) / (dev_ms / 1000.0) / n / 1e12,
               "impl": "library",
               "library": "torch %s: F.linear (cuBLAS), %s, F.layer_norm, AdamW(fused), NCCL" % (
                   torch.__version__, "flash_attn_func" if la._flash is not None else "F.scaled_dot_product_attention"),
               "config": {"model": args.model, "global_batch": global_batch, "seq_len": seq, "micro_batch": micro,
                          "grad_accum": gas, "parallelism": f"tp{tp}" + ("+sp" if tp > 1 else "") + f" x dp{dp}, zero1",
                          "l2": "working set far exceeds the 126 MB L2; no explicit flush"},
               "clocks": clocks, "e2e": e2e, "gpu_launches": 0}
        print(json.dumps(out))
        if args.json_out:
            with open(args.json_out, "w") as f:
                f.write(json.dumps(out) + "\n")
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def neox_20b_children(args, rank, local_rank):
    """The second headline configuration, measured after the main run in one fresh child process per rank
    (the parent has left its process group and released its device memory).  Rank 0 returns the child's
    JSON line as a dict; a failure is reported as {"unavailable": reason}, never raised."""
    import tempfile
    out_path = os.path.join(tempfile.gettempdir(), f"neox20b_bench_{os.environ.get('MASTER_PORT', '0')}.json")
    env = dict(os.environ)
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29511")) + 17)
    for k in ("TORCHELASTIC_RUN_ID", "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS",
              "TORCHELASTIC_USE_AGENT_STORE", "TORCH_NCCL_ASYNC_ERROR_HANDLING"):
        env.pop(k, None)
    cmd = [sys.executable, os.path.abspath(__file__), "--gpus", "8", "--model", "neox-20B", "--steps",
           "10", "--warmup", "3", "--mode", args.mode, "--no-20b",
           "--json-out", out_path]
    try:
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
        if rank != 0:
            return None
        if r.returncode != 0 or not os.path.exists(out_path):
            tail = (r.stderr or r.stdout or "").strip().splitlines()[-3:]
            return {"unavailable": f"child exited {r.returncode}: " + " | ".join(tail)}
        with open(out_path) as f:
            d = json.loads(f.read())
        os.remove(out_path)
        keep = ("value", "unit", "ms_per_step", "tflops_per_gpu", "steps", "warmup", "e2e", "config", "clocks",
                "gpu_launches", "device_error_word")
        return {k: d.get(k) for k in keep}
    except Exception as e:  # noqa: BLE001 - the main number must be printed whatever happens here
        return {"unavailable": f"{type(e).__name__}: {e}"} if rank == 0 else None


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "library":
        return library_arm(args)
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n = args.gpus
    assert world == n or world == 1 and n == 1, f"--gpus {n} but WORLD_SIZE={world}: launch with torchrun"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")

    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.data.data_utils import build_train_valid_test_data_loaders, shift_and_wrap_data_loaders
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.obs.logging import get_flops
    from gpt_neox_b200.ops.gemm import LAUNCHES
    from gpt_neox_b200.utils.common import Timers

    pp = 1
    if "20B" in args.model:
        # the named NeoX-20B configuration: TP 4 x PP 2 on 8 GPUs, micro-batch 2, 16 micro-batches per step
        assert n == 8, "the NeoX-20B benchmark layout (tp4 x pp2) needs --gpus 8"
        tp, pp = 4, 2
        dp = n // (tp * pp)
        micro = args.micro_batch or 2
        gas = args.gas or 16
        global_batch = micro * gas * dp
    elif "dmoe" in args.model:
        # 125M dropless MoE: expert parallel over all GPUs (8 experts), micro-batch 8, one micro-batch per step
        tp, dp = 1, n
        assert 8 % n == 0, "the dMoE benchmark shards 8 experts over the GPUs"
        micro = args.micro_batch or 8
        gas = args.gas or 1
        global_batch = micro * gas * dp
    else:
        # Pythia-6.9B: the named layout is TP 2 (+ sequence parallelism) x DP N/2; Pythia-1.4B: pure data parallel
        tp = 1 if (n == 1 or "1-4B" in args.model) else 2
        dp = n // tp
        micro = args.micro_batch or (4 if "6-9B" in args.model else 16)
        per_gpu_seqs = 64 if "6-9B" in args.model else 128         # sequences per GPU per optimizer step
        global_batch = per_gpu_seqs * n
        gas = args.gas or global_batch // (micro * dp)
        global_batch = micro * gas * dp
    total_iters = args.warmup + 2 * args.steps + 4
    over = {"global_num_gpus": n, "model_parallel_size": tp, "pipe_parallel_size": pp if pp > 1 else 0,
            "sequence_parallel": tp > 1,
            "train_micro_batch_size_per_gpu": micro, "gradient_accumulation_steps": gas, "train_batch_size": None,
            "comm_mode": args.mode, "train_iters": total_iters, "lr_decay_iters": 143000, "log_interval": 10 ** 9,
            "make_vocab_size_divisible_by": 128 if tp <= 2 else 64}
    if "dmoe" in args.model:
        over["moe_expert_parallel_size"] = n
    if args.fp8:
        over.update(te_columnparallel=True, te_rowparallel=True, te_fp8_amax_history_len=16,
                    te_fp8_amax_compute_algo="max", te_fp8_recipe=args.fp8_recipe)
        if tp > 1:
            over["comm_mode"] = "nccl_baseline"      # the fused AG/RS GEMM kernels are bf16
    neox_args = NeoXArgs.from_ymls([os.path.join(REPO, "configs", "bench", args.model + ".yml")], overwrite_values=over)
    neox_args.configure_distributed_args()
    neox_args.build_tokenizer()
    neox_args.initialize_tensorboard_writer()
    initialize_megatron(neox_args)
    timers = Timers(use_wandb=False, tensorboard_writer=None)
    model, optimizer, lr_scheduler, _ = training.setup_model_and_optimizer(neox_args=neox_args, use_cache=False)
    model.train()
    dev = torch.device("cuda", torch.cuda.current_device())
    seq = neox_args.seq_length

    # ---- device-resident batches for the kernel-timed region (distinct data per data-parallel rank)
    g = torch.Generator(device="cpu")
    g.manual_seed(1234 + mpu.get_data_parallel_rank())
    pool = [{"text": torch.randint(0, 50277, (micro, seq + 1), generator=g, dtype=torch.int64).to(dev)}
            for _ in range(min(gas, 8))]

    def device_iter():
        i = 0
        while True:
            yield pool[i % len(pool)]
            i += 1

    def barrier_sync():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run_steps(it, k, read_loss):
        last = None
        for _ in range(k):
            loss_dict, _skipped = training.train_step(neox_args=neox_args, timers=timers, data_iterator=it,
                                                      model=model, optimizer=optimizer, lr_scheduler=lr_scheduler)
            if read_loss:
                last = float(loss_dict["lm_loss"].item())       # device -> host read every step
            neox_args.iteration += 1
        return last

    dit = device_iter()
    run_steps(dit, args.warmup, read_loss=False)
    sampler = ClockSampler(local_rank)
    barrier_sync()
    if rank == 0:
        sampler.start()
    l0 = LAUNCHES["n"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t_enq = time.perf_counter()
    run_steps(dit, args.steps, read_loss=False)
    enqueue_ms = (time.perf_counter() - t_enq) * 1000.0 / args.steps     # host time to issue one step's work
    e1.record()
    barrier_sync()
    launches = LAUNCHES["n"] - l0
    clocks = sampler.stop() if rank == 0 else None
    dev_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    loss_now = float(training.reduce_losses([torch.zeros((), device=dev)]).item())  # keeps collectives aligned
    del loss_now

    # ---- end to end: the framework's own loader (pinned host memory -> device per micro-batch),
    #      loss read back every step
    e2e = None
    if not args.no_e2e:
        loaders = build_train_valid_test_data_loaders(neox_args=neox_args)
        train_it, _, _ = shift_and_wrap_data_loaders(neox_args=neox_args, data_loaders=loaders)
        run_steps(train_it, 1, read_loss=True)
        barrier_sync()
        t0 = time.perf_counter()
        last_loss = run_steps(train_it, args.steps, read_loss=True)
        barrier_sync()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1000.0) / args.steps
        tokens = global_batch * seq
        e2e = {"value": tokens / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": gas * micro * (seq + 1) * 8, "d2h_bytes_per_step": 4,
               "final_loss": last_loss}

    if args.kernel_table:
        from torch.profiler import ProfilerActivity, profile
        barrier_sync()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            run_steps(dit, 1, read_loss=False)
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.kernel_table, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=60, max_name_column_width=90))

    from gpt_neox_b200.ops import _lib
    dev_err = _lib.read_device_error(clear=False)
    if rank == 0:
        tokens = global_batch * seq
        tps = tokens / (dev_ms / 1000.0)
        neox_args.train_batch_size = global_batch
        tflops = get_flops(neox_args, dev_ms / 1000.0, use_checkpointing_factor=False) / 1e12
        if "dmoe" in args.model:
            # the dense formula counts one FFN per token; a top-k MoE layer runs k expert FFNs (active-parameter FLOPs)
            ffn = neox_args.intermediate_size or 4 * neox_args.hidden_size
            extra = 3 * 4.0 * neox_args.hidden_size * ffn * (neox_args.moe_top_k - 1) * neox_args.num_layers * tokens
            tflops += extra / (dev_ms / 1000.0) / n / 1e12
        out = {"metric": "tokens_per_sec", "value": tps, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": ("fp8" if args.fp8_recipe == "delayed" else "mxfp8") if args.fp8 else "bf16", "data": "synthetic tokens, random-init weights",
               "tflops_per_gpu": tflops, "impl": "ours", "mode": args.mode,
               "config": {"model": args.model, "global_batch": global_batch, "seq_len": seq, "micro_batch": micro,
                          "grad_accum": gas,
                          "parallelism": (f"tp{tp}" + ("+sp" if tp > 1 else "") + (f" x pp{pp}" if pp > 1 else "")
                                          + f" x dp{dp}, zero1" + (f", ep{n}" if "dmoe" in args.model else "")),
                          "l2": "working set (weights + activations, tens of GB) far exceeds the 126 MB L2; "
                                "no explicit flush"},
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "host_enqueue_ms_per_step": enqueue_ms, "device_error_word": dev_err}
    with_20b = (n == 8 and args.model == "pythia-6-9B" and not args.no_20b and not args.fp8
                and os.environ.get("NEOX_BENCH_20B", "1") != "0")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    if with_20b:
        # release this process's device memory, then measure GPT-NeoX-20B (tp4 x pp2) in child processes
        del model, optimizer, lr_scheduler, pool, dit
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        extra = neox_20b_children(args, rank, local_rank)
        if rank == 0:
            out["neox_20b"] = extra
    if rank == 0:
        print(json.dumps(out))
        if args.json_out:
            with open(args.json_out, "w") as f:
                f.write(json.dumps(out) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
