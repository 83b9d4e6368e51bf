"""Checkpoint save / resume: bit-equal parameters, identical continued loss curve, data-parallel resize of the
ZeRO shards, and handling of damaged checkpoints (reference: tests/model/test_model_checkpoint.py)."""
import os

import pytest
import torch

from common import run_distributed, tiny_config


def _train(rank, world, cfg, steps, start_from=None):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    cfg = dict(cfg, global_num_gpus=world, train_iters=steps)
    a = NeoXArgs.from_dict(cfg)
    a.configure_distributed_args()
    a.build_tokenizer()
    losses = []
    training.collect_loss_for_unit_test = lambda l: losses.append(float(l))
    training.pretrain(a)
    return losses


def _cfg(tmp, **over):
    return tiny_config(use_cpu_initialization=True, save=str(tmp), load=str(tmp), checkpoint_factor=4,
                       lr_decay_iters=8, **over)


def test_resume_continues_the_uninterrupted_run(tmp_path):
    full = run_distributed(_train, 1, _cfg(tmp_path / "a"), 8)[0]
    first = run_distributed(_train, 1, _cfg(tmp_path / "b"), 4)[0]
    assert first == pytest.approx(full[:4], rel=1e-6)
    assert os.path.isdir(tmp_path / "b" / "global_step4") and (tmp_path / "b" / "latest").read_text().strip() == "global_step4"
    rest = run_distributed(_train, 1, _cfg(tmp_path / "b"), 8)[0]          # picks up at iteration 4
    assert len(rest) == 4
    assert rest == pytest.approx(full[4:], rel=1e-5)


def test_zero_shards_are_repartitioned_when_the_data_parallel_size_changes(tmp_path):
    """Saved by 2 data-parallel ranks (two optimizer shards), resumed by 1: same curve as a 1-rank run."""
    two = _cfg(tmp_path / "c", train_micro_batch_size_per_gpu=2)
    one = _cfg(tmp_path / "c", train_micro_batch_size_per_gpu=4)
    ref = run_distributed(_train, 1, _cfg(tmp_path / "ref", train_micro_batch_size_per_gpu=4), 8)[0]
    first = run_distributed(_train, 2, two, 4)[0]
    assert first == pytest.approx(ref[:4], rel=2e-5)
    files = os.listdir(tmp_path / "c" / "global_step4")
    assert sum("optim_states" in f for f in files) == 2
    rest = run_distributed(_train, 1, one, 8)[0]
    assert rest == pytest.approx(ref[4:], rel=1e-4)


def test_damaged_checkpoints(tmp_path):
    from gpt_neox_b200.ckpt import io
    d = tmp_path / "d"
    run_distributed(_train, 1, _cfg(d), 4)
    # an interrupted save leaves only a .tmp directory: it is never taken for a checkpoint
    os.makedirs(d / "global_step8.tmp")
    assert io.read_latest_tag(str(d)) == "global_step4"
    # a `latest` file that names a missing tag is an explicit error, not a silent fresh start
    (d / "latest").write_text("global_step999")
    with pytest.raises(Exception):
        run_distributed(_train, 1, _cfg(d), 8)
    # a truncated model-state file fails loudly as well
    (d / "latest").write_text("global_step4")
    f = d / "global_step4" / "mp_rank_00_model_states.pt"
    data = f.read_bytes()
    f.write_bytes(data[: len(data) // 2])
    with pytest.raises(Exception):
        run_distributed(_train, 1, _cfg(d), 8)


@pytest.mark.parametrize("world,over", [
    (2, dict(moe_num_experts=4, moe_top_k=2, gpt_j_residual=False, moe_router_type="topk", moe_expert_parallel_size=2)),
    (1, dict(optimizer={"type": "sm3", "params": {"lr": 1e-3}})),
    (1, dict(gradient_accumulation_steps=2, hidden_dropout=0.1)),
    (2, dict(use_bnb_optimizer=True)),
    (2, dict(zero_optimization={"stage": 3})),
    (1, dict(attention_dropout=0.1, attention_config=[[["flash"], 2]], checkpoint_activations=True)),
], ids=["moe_expert_parallel_2", "sm3_state", "dropout_rng", "adam_8bit_state", "zero_stage3", "attention_dropout_recompute"])
def test_resume_is_exact_for_expert_parallel_generic_optimizer_and_dropout(tmp_path, world, over):
    """Things a resume has to carry beyond the dense weights and Adam moments: the experts of every expert-parallel
    rank (one state file per rank), the own state of SM3 / MADGRAD / Lion / SGD, and the random streams (re-applied
    after the data iterators are rebuilt, which draw from them)."""
    full = run_distributed(_train, world, _cfg(tmp_path / "a", **over), 8)[0]
    first = run_distributed(_train, world, _cfg(tmp_path / "b", **over), 4)[0]
    rest = run_distributed(_train, world, _cfg(tmp_path / "b", **over), 8)[0]
    assert first == pytest.approx(full[:4], rel=1e-6)
    assert len(rest) == 4 and rest == pytest.approx(full[4:], rel=2e-5)
    if "moe_expert_parallel_size" in over:
        files = os.listdir(tmp_path / "b" / "global_step8")
        assert sum(f.startswith("expert_ep_rank_") for f in files) == 2
