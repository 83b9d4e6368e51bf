"""Shared test helpers: tiny configs and a spawn-N-processes harness with a wall-clock guard."""
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def tiny_config(**over):
    cfg = dict(num_layers=2, hidden_size=64, num_attention_heads=4, seq_length=32, max_position_embeddings=32,
               pos_emb="rotary", rotary_pct=0.25, gpt_j_residual=True, no_weight_tying=True, norm="layernorm",
               attention_config=[[["global"], 2]], train_micro_batch_size_per_gpu=2, gradient_accumulation_steps=1,
               optimizer={"type": "Adam", "params": {"lr": 6e-4, "betas": [0.9, 0.95], "eps": 1e-8}},
               precision="fp32", train_iters=10, lr_decay_iters=10, dataset_impl="synthetic",
               synthetic_vocab_size=100, tokenizer_type="HFTokenizer", zero_optimization={"stage": 1},
               global_num_gpus=1, log_interval=1000, init_method="normal", output_layer_init_method="normal",
               distributed_backend="gloo", num_workers=0, eval_interval=1000, eval_iters=1, weight_decay=0.01,
               gradient_clipping=1.0)
    cfg.update(over)
    if "num_layers" in over and "attention_config" not in over:
        cfg["attention_config"] = [[["global"], cfg["num_layers"]]]
    return cfg


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world))
    try:
        ret[rank] = ("ok", fn(rank, world, *args))
    except BaseException as e:  # noqa: BLE001 - report every failure of a child to the parent
        ret[rank] = ("err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}")


def run_distributed(fn, world_size, *args, timeout=240):
    """Run ``fn(rank, world, *args)`` in ``world_size`` spawned CPU processes; return their results.
    A child that does not finish within ``timeout`` seconds is killed (exact PIDs) and the test fails."""
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, args, ret)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    assert not hung, f"{len(hung)} rank(s) hung for more than {timeout}s"
    out, errors = [], []
    for r in range(world_size):
        status, val = ret.get(r, ("err", "no result (process died)"))
        if status != "ok":
            errors.append(f"--- rank {r} failed:\n{val}")
        out.append(val)
    # a rank that dies takes its peers' connections down: show the failure that is not a lost connection first
    errors.sort(key=lambda e: "Connection closed by peer" in e or "Connection reset" in e)
    assert not errors, "\n".join(errors)
    return out
