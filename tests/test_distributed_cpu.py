"""Parallel algebra on CPU (gloo): tensor / sequence parallel and ZeRO-1 data parallel runs must
reproduce the single-process loss curve."""
import pytest
import torch

from common import run_distributed, tiny_config

pytestmark = pytest.mark.cpu


def _train(rank, world, cfg, steps):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    cfg = dict(cfg, global_num_gpus=world, train_iters=steps, lr_decay_iters=steps)
    a = NeoXArgs.from_dict(cfg)
    a.configure_distributed_args()
    a.build_tokenizer()
    losses = []
    training.collect_loss_for_unit_test = lambda l: losses.append(float(l))
    training.pretrain(a)
    return losses


def _train_with_norms(rank, world, cfg, steps):
    """As _train, but also returns the global gradient norm the engine reports after every step."""
    from gpt_neox_b200 import training
    norms = []
    orig = training.train_step

    def wrapped(*a, **kw):
        out = orig(*a, **kw)
        norms.append(kw["model"].get_global_grad_norm())
        return out
    training.train_step = wrapped
    try:
        return _train(rank, world, cfg, steps), norms
    finally:
        training.train_step = orig


def _single(cfg, steps):
    return run_distributed(_train, 1, cfg, steps)[0]


def test_config1_plumbing_zero1_dp2_matches_single_process():
    """19M-style decoder (scaled down), world 2, ZeRO-1, fp32, 10 AdamW steps: loss decreases and equals
    the one-process run to reduction-order noise."""
    cfg = tiny_config(num_layers=3, hidden_size=64, num_attention_heads=4, seq_length=64, max_position_embeddings=64,
                      train_batch_size=4, train_micro_batch_size_per_gpu=None, gradient_accumulation_steps=1,
                      use_cpu_initialization=True)
    ref = _single(dict(cfg, train_micro_batch_size_per_gpu=4, train_batch_size=None), 10)
    cfg2 = dict(cfg, train_micro_batch_size_per_gpu=2, train_batch_size=None)
    out = run_distributed(_train, 2, cfg2, 10)
    assert out[0] == pytest.approx(out[1], rel=1e-6)
    assert out[0] == pytest.approx(ref, rel=2e-5)
    assert min(ref[5:]) < ref[0]


@pytest.mark.parametrize("layout", ["dp2", "pp2_dp2"])
def test_zero_stage0_grad_norm_and_clipping_match_single_process(layout):
    """Without ZeRO sharding every data-parallel rank holds the whole reduced gradient: the global norm must
    count it once, not once per rank.  Clipping is set low enough to bite on every step, so a wrong norm
    would change the loss curve too."""
    cfg = tiny_config(use_cpu_initialization=True, zero_optimization={"stage": 0}, gradient_clipping=0.05,
                      num_layers=4, train_micro_batch_size_per_gpu=4, gradient_accumulation_steps=2)
    pp = {"pipe_parallel_size": 2} if layout == "pp2_dp2" else {}
    ref, ref_norms = run_distributed(_train_with_norms, 2 if pp else 1, dict(cfg, **pp), 4)[0]
    out = run_distributed(_train_with_norms, 4 if pp else 2, dict(cfg, train_micro_batch_size_per_gpu=2, **pp), 4)
    losses, norms = out[0]
    assert min(ref_norms) > 0.05                       # the clip is active
    assert norms == pytest.approx(ref_norms, rel=1e-4)
    assert losses == pytest.approx(ref, rel=5e-5)


@pytest.mark.parametrize("sp", [False, True])
def test_tensor_parallel_2_matches_tp1(sp):
    # the vocabulary is padded to a multiple of divisible_by x tp: 256 in both runs.  Row-parallel
    # biases are off: under the GPT-J residual they are added on every rank before the reduction
    # (effective bias = tp x bias, the convention the checkpoint converters compensate for), so a
    # TP-2 run with them is by design not the TP-1 run.
    cfg = tiny_config(use_cpu_initialization=True, train_micro_batch_size_per_gpu=2, make_vocab_size_divisible_by=256,
                      use_bias_in_attn_linear=False, use_bias_in_mlp=False)
    ref = _single(cfg, 4)
    out = run_distributed(_train, 2, dict(cfg, model_parallel_size=2, sequence_parallel=sp,
                                          make_vocab_size_divisible_by=128), 4)
    assert out[0] == pytest.approx(out[1], rel=1e-6)
    assert out[0] == pytest.approx(ref, rel=5e-5)


def test_tp2_sequential_residual_rmsnorm():
    # (GQA and gated MLPs shard [Q|K|V] / [value|gate] blocks per rank, so a TP-2 model is not the
    #  row-for-row split of the TP-1 master; they are covered by the single-rank oracle tests.)
    cfg = tiny_config(use_cpu_initialization=True, gpt_j_residual=False, norm="rmsnorm",
                      make_vocab_size_divisible_by=256)
    ref = _single(cfg, 3)
    out = run_distributed(_train, 2, dict(cfg, model_parallel_size=2, sequence_parallel=True,
                                          make_vocab_size_divisible_by=128), 3)
    assert out[0] == pytest.approx(ref, rel=5e-5)


def test_tp2_x_dp2_world4():
    cfg = tiny_config(use_cpu_initialization=True, train_micro_batch_size_per_gpu=2, make_vocab_size_divisible_by=256,
                      use_bias_in_attn_linear=False, use_bias_in_mlp=False)
    ref = _single(dict(cfg, train_micro_batch_size_per_gpu=4), 3)
    out = run_distributed(_train, 4, dict(cfg, model_parallel_size=2, sequence_parallel=True,
                                          make_vocab_size_divisible_by=128), 3)
    assert out[0] == pytest.approx(ref, rel=5e-5)


def test_pipeline_parallel_2_matches_sequential():
    """1F1B over two stages (4 micro-batches) reproduces the unpipelined loss curve."""
    cfg = tiny_config(use_cpu_initialization=True, num_layers=4, train_micro_batch_size_per_gpu=2,
                      gradient_accumulation_steps=4)
    ref = _single(cfg, 4)
    out = run_distributed(_train, 2, dict(cfg, pipe_parallel_size=2), 4)
    assert out[0] == pytest.approx(out[1], rel=1e-6)
    assert out[0] == pytest.approx(ref, rel=5e-5)


def test_pipeline_2_x_tensor_2_with_tied_embeddings():
    cfg = tiny_config(use_cpu_initialization=True, num_layers=4, train_micro_batch_size_per_gpu=2,
                      gradient_accumulation_steps=2, no_weight_tying=False, make_vocab_size_divisible_by=256,
                      use_bias_in_attn_linear=False, use_bias_in_mlp=False)
    ref = _single(cfg, 3)
    out = run_distributed(_train, 4, dict(cfg, pipe_parallel_size=2, model_parallel_size=2,
                                          make_vocab_size_divisible_by=128), 3)
    assert out[0] == pytest.approx(ref, rel=5e-5)


@pytest.mark.parametrize("gpt_j", [False, True])
def test_moe_expert_parallel_2_matches_single_rank(gpt_j):
    """Dropless MoE with all-to-all dispatch over 2 expert-parallel ranks == the single-rank MoE, for the
    sequential and the parallel (GPT-J) residual form."""
    cfg = tiny_config(use_cpu_initialization=True, gpt_j_residual=gpt_j, moe_num_experts=4, moe_top_k=2,
                      moe_router_type="topk", moe_expert_interval=1, train_micro_batch_size_per_gpu=2)
    ref = _single(dict(cfg, train_micro_batch_size_per_gpu=4), 3)
    out = run_distributed(_train, 2, dict(cfg, moe_expert_parallel_size=2), 3)
    assert out[0] == pytest.approx(out[1], rel=1e-6)
    assert out[0] == pytest.approx(ref, rel=1e-4)


def test_t5_relative_position_bias_tp2_pp2_match_single_rank():
    """``pos_emb: rpe``: one bucketed bias table per rank shared by its layers, heads sharded over tensor
    parallel.  The shared table receives the gradients of every layer (the loss falls) and the TP-2 run
    reproduces the TP-1 losses."""
    cfg = tiny_config(use_cpu_initialization=True, pos_emb="rpe", rpe_num_buckets=8, rpe_max_distance=16,
                      make_vocab_size_divisible_by=256, use_bias_in_attn_linear=False, use_bias_in_mlp=False)
    ref = _single(cfg, 6)
    assert ref[-1] < ref[0]
    out = run_distributed(_train, 2, dict(cfg, model_parallel_size=2, make_vocab_size_divisible_by=128), 6)
    assert out[0] == pytest.approx(ref, rel=5e-5)


def test_partitioned_and_offloaded_activation_checkpoints_tp2():
    """``partition_activations`` keeps 1/tp of every checkpointed layer input per rank (re-assembled by an
    all-gather in backward) and ``checkpoint_in_cpu`` parks it in host memory: the losses are those of plain
    activation checkpointing, with and without sequence parallelism (where the inputs are sharded already)."""
    cfg = tiny_config(use_cpu_initialization=True, model_parallel_size=2, make_vocab_size_divisible_by=128,
                      checkpoint_activations=True, checkpoint_num_layers=1)
    ref = run_distributed(_train, 2, cfg, 3)[0]
    got = run_distributed(_train, 2, dict(cfg, partition_activations=True, checkpoint_in_cpu=True,
                                          synchronize_each_layer=True), 3)[0]
    assert got == pytest.approx(ref, rel=1e-6)
    sp = run_distributed(_train, 2, dict(cfg, sequence_parallel=True), 3)[0]
    got = run_distributed(_train, 2, dict(cfg, sequence_parallel=True, partition_activations=True), 3)[0]
    assert got == pytest.approx(sp, rel=1e-6)


def _stash_sizes(rank, world):
    import torch.distributed as dist
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200.parallel import random as prandom
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mpu.destroy_model_parallel()
    mpu.initialize_model_parallel(2)
    prandom.configure_checkpointing(partition_activations=True)
    x = torch.arange(24, dtype=torch.float32).view(4, 6).requires_grad_(True)
    mask = torch.ones(4, 4, dtype=torch.bool)
    kept = prandom._stash(x)
    back = prandom._unstash(kept)
    out = (kept[0], kept[1].numel(), prandom._stash(mask)[0], bool(torch.equal(back, x)), back.requires_grad)
    prandom.configure_checkpointing()
    dist.destroy_process_group()
    return out


def test_activation_stash_keeps_one_slice_per_rank():
    for r in run_distributed(_stash_sizes, 2):
        assert r == ("slice", 12, "full", True, True)


@pytest.mark.parametrize("gpt_j", [False, True])
def test_moe_under_tensor_and_sequence_parallelism_matches_tp1(gpt_j):
    """MoE routers and experts are replicated over the tensor-parallel group; under sequence parallelism each
    rank routes only its part of the sequence, so their gradients are summed over the group (a second step
    that differs from TP-1 is the symptom when they are not)."""
    cfg = tiny_config(use_cpu_initialization=True, gpt_j_residual=gpt_j, moe_num_experts=4, moe_top_k=2,
                      moe_router_type="topk", moe_expert_interval=1, make_vocab_size_divisible_by=256,
                      use_bias_in_attn_linear=False, use_bias_in_mlp=False)
    ref = _single(cfg, 3)
    out = run_distributed(_train, 2, dict(cfg, model_parallel_size=2, sequence_parallel=True,
                                          make_vocab_size_divisible_by=128), 3)[0]
    assert out == pytest.approx(ref, rel=2e-6)


def test_qk_layernorm_is_not_summed_over_the_group_under_sequence_parallelism():
    """The QK norm works on this rank's heads of the full sequence, so sequence parallelism must leave its
    gradients alone: TP-2 with and without sequence parallelism train identically."""
    cfg = tiny_config(use_cpu_initialization=True, model_parallel_size=2, make_vocab_size_divisible_by=128,
                      use_qk_layernorm=True, gpt_j_residual=False)
    a = run_distributed(_train, 2, cfg, 4)[0]
    b = run_distributed(_train, 2, dict(cfg, sequence_parallel=True), 4)[0]
    assert b == pytest.approx(a, rel=2e-6)


def _train_stage3(rank, world, cfg, steps):
    """As _train; also reports how many parameter elements each rank holds between steps and after a gather."""
    from gpt_neox_b200 import training
    held = {}
    orig = training.train_step

    def wrapped(*a, **kw):
        out = orig(*a, **kw)
        eng = kw["model"]
        held["between_steps"] = sum(p.data.numel() for p in eng.module.parameters())
        held["slices"] = sum(g.lp_shard.numel() for g in eng.groups if g.partition_params)
        held["total"] = eng.total_params
        held["groups"] = len(eng.groups)
        return out
    training.train_step = wrapped
    try:
        return _train(rank, world, cfg, steps), held
    finally:
        training.train_step = orig


@pytest.mark.parametrize("over", [dict(), dict(checkpoint_activations=True, checkpoint_num_layers=1),
                                  dict(no_weight_tying=False, gradient_accumulation_steps=2)],
                         ids=["plain", "activation_checkpointing", "tied_embeddings_gas2"])
def test_zero_stage3_partitions_parameters_and_matches_stage1(over):
    """ZeRO stage 3 over two data-parallel ranks: each layer's parameters are gathered for its forward and backward
    and dropped afterwards (between steps a rank holds no gathered parameter, only its slices: about half the
    model), gradients are reduce-scattered per layer, and the loss curve is the stage-1 curve."""
    cfg = tiny_config(use_cpu_initialization=True, num_layers=3, train_micro_batch_size_per_gpu=2, **over)
    ref = run_distributed(_train, 2, cfg, 5)[0]
    out = run_distributed(_train_stage3, 2, dict(cfg, zero_optimization={"stage": 3}), 5)
    (losses, held), (losses1, _) = out
    assert losses == pytest.approx(losses1, rel=1e-6)
    assert losses == pytest.approx(ref, rel=2e-5)
    assert held["between_steps"] == 0 and held["groups"] >= 5
    assert held["total"] / 2 <= held["slices"] < held["total"] / 2 + 256 * 2 * held["groups"]


def _train_overlap(rank, world, cfg, steps):
    """As _train; also counts the ranges started from inside the backward pass (before the step's own reduction)."""
    from gpt_neox_b200.engine import engine as eng
    started = {"in_backward": 0, "at_step": 0, "in_step": False}
    orig_async, orig_finish = eng.FlatGroup.reduce_range_async, eng.FlatGroup._finish_bucketed

    def counting(self, lo, hi):
        started["at_step" if started["in_step"] else "in_backward"] += 1
        return orig_async(self, lo, hi)

    def finishing(self):
        started["in_step"] = True
        try:
            return orig_finish(self)
        finally:
            started["in_step"] = False
    eng.FlatGroup.reduce_range_async, eng.FlatGroup._finish_bucketed = counting, finishing
    try:
        return _train(rank, world, cfg, steps), started
    finally:
        eng.FlatGroup.reduce_range_async, eng.FlatGroup._finish_bucketed = orig_async, orig_finish


@pytest.mark.parametrize("over", [dict(), dict(checkpoint_activations=True, checkpoint_num_layers=1),
                                  dict(no_weight_tying=False, gradient_accumulation_steps=2, gradient_clipping=0.05),
                                  dict(zero_optimization={"stage": 0, "overlap_comm": True}, prescale_gradients=True)],
                         ids=["plain", "activation_checkpointing", "tied_embeddings_gas2_clip", "stage0_prescale"])
def test_gradient_reduction_overlapped_with_backward_matches_the_single_reduction(over):
    """``overlap_comm``: every layer's gradients are reduced from inside the backward pass of the last micro-batch
    (one bucket per layer, nothing but leftovers at the step) and the loss curve is that of the single reduction."""
    cfg = tiny_config(use_cpu_initialization=True, num_layers=3, train_micro_batch_size_per_gpu=2,
                      zero_optimization={"stage": 1, "overlap_comm": False})
    cfg.update(over)
    zo = dict(cfg["zero_optimization"])
    ref = run_distributed(_train, 2, dict(cfg, zero_optimization=dict(zo, overlap_comm=False)), 5)[0]
    out = run_distributed(_train_overlap, 2, dict(cfg, zero_optimization=dict(zo, overlap_comm=True)), 5)
    (losses, started), (losses1, _) = out
    assert losses == pytest.approx(losses1, rel=1e-6)
    assert losses == pytest.approx(ref, rel=1e-6)
    assert started["in_backward"] >= 5 * 5              # embedding, three layers, final norm (+ read-out) per step
    assert started["at_step"] <= 5 * 2                  # alignment tails only
