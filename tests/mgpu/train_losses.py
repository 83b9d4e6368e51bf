"""Run a few training steps of a small model on the visible GPUs (launched by torchrun) and print the
loss curve as JSON on rank 0.  Used by the multi-GPU tests to compare communication modes."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    mode, tp, sp, steps = sys.argv[1], int(sys.argv[2]), sys.argv[3] == "1", int(sys.argv[4])
    extra = json.loads(sys.argv[5]) if len(sys.argv) > 5 else {}
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.ops import _lib
    from gpt_neox_b200.utils.common import Timers
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = dict(num_layers=4, hidden_size=1024, num_attention_heads=8, seq_length=512, max_position_embeddings=512,
               pos_emb="rotary", rotary_pct=0.25, gpt_j_residual=True, no_weight_tying=True, norm="layernorm",
               attention_config=[[["flash"], 4]], train_micro_batch_size_per_gpu=4, gradient_accumulation_steps=2,
               optimizer={"type": "Adam", "params": {"lr": 1e-3, "betas": [0.9, 0.95], "eps": 1e-8}},
               precision="bfloat16", train_iters=steps, lr_decay_iters=steps, dataset_impl="synthetic",
               synthetic_vocab_size=4000, tokenizer_type="HFTokenizer", zero_optimization={"stage": 1},
               global_num_gpus=world, log_interval=1000, init_method="normal", output_layer_init_method="normal",
               num_workers=0, eval_interval=1000, eval_iters=1, model_parallel_size=tp, sequence_parallel=sp,
               comm_mode=mode, make_vocab_size_divisible_by=128)
    cfg.update(extra)
    a = NeoXArgs.from_dict(cfg)
    a.configure_distributed_args()
    a.build_tokenizer()
    initialize_megatron(a)
    model, opt, sched, _ = training.setup_model_and_optimizer(neox_args=a, use_cache=False)
    model.train() if hasattr(model, "train") else None
    from gpt_neox_b200 import parallel as mpu
    g = torch.Generator().manual_seed(7 + mpu.get_data_parallel_rank())
    batches = [{"text": torch.randint(0, 4000, (4, 513), generator=g).cuda()} for _ in range(4)]

    def it():
        i = 0
        while True:
            yield batches[i % 4]
            i += 1
    data, timers, losses = it(), Timers(), []
    for _ in range(steps):
        ld, _ = training.train_step(neox_args=a, timers=timers, data_iterator=data, model=model, optimizer=opt,
                                    lr_scheduler=sched)
        losses.append(float(ld["lm_loss"].item()))
    err = _lib.read_device_error()
    if int(os.environ.get("RANK", "0")) == 0:
        zs = any(getattr(g, "zero_ws", None) is not None for g in getattr(model, "groups", []))
        from gpt_neox_b200.comm import symm
        tp_be = symm.backend_for(mpu.get_model_parallel_group())
        calls = {k: getattr(tp_be, k, 0) for k in ("ag_calls", "rs_calls", "ar_calls")} if tp_be is not None else {}
        from gpt_neox_b200.ops import moe_ep
        buckets = int(getattr(model, "_ov_buckets", 0))
        pool = getattr(tp_be, "pool", None) if tp_be is not None else None
        print("LOSSES " + json.dumps({"losses": losses, "device_error": err, "zero_symm": zs, "fused_calls": calls,
                                      "overlap_buckets": buckets, "gather_pool_slots": pool["n"] if pool else 0,
                                      "moe_p2p": bool(moe_ep._WORKSPACES)}),
              flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
