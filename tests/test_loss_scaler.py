"""fp16 loss scaling: the dynamic scaler's schedule and the engine skipping a step on overflow
(reference behaviour: DeepSpeed's DynamicLossScaler driven by the `fp16` config block)."""
import pytest
import torch

from common import run_distributed, tiny_config
from gpt_neox_b200.engine.loss_scaler import DynamicLossScaler, LossScaler, build_loss_scaler


def test_static_and_dynamic_construction():
    s = build_loss_scaler({"loss_scale": 128})
    assert isinstance(s, LossScaler) and not s.dynamic and s.cur_scale == 128.0
    d = build_loss_scaler({"loss_scale": 0, "initial_scale_power": 12, "loss_scale_window": 4, "hysteresis": 2,
                           "min_loss_scale": 1})
    assert isinstance(d, DynamicLossScaler) and d.cur_scale == 4096.0


def test_dynamic_scaler_schedule():
    d = DynamicLossScaler(init_scale=1024, scale_window=3, min_scale=64, hysteresis=2)
    d.update_scale(True)                  # first overflow is absorbed by the hysteresis
    assert d.cur_scale == 1024
    d.update_scale(True)                  # second one halves
    assert d.cur_scale == 512
    for _ in range(2):
        d.update_scale(False)
    assert d.cur_scale == 512
    d.update_scale(False)                 # third clean step since the overflow: double
    assert d.cur_scale == 1024
    for _ in range(20):                   # never below the floor
        d.update_scale(True)
    assert d.cur_scale == 64
    sd = d.state_dict()
    e = DynamicLossScaler(init_scale=1, scale_window=3, min_scale=64, hysteresis=2)
    e.load_state_dict(sd)
    assert e.cur_scale == 64 and e.cur_iter == d.cur_iter


def _train(rank, world, cfg, steps):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world, train_iters=steps))
    a.configure_distributed_args()
    a.build_tokenizer()
    losses = []
    training.collect_loss_for_unit_test = lambda l: losses.append(float(l))
    model = training.pretrain(a)
    return {"losses": losses, "skipped": model.skipped_steps, "scale": model.loss_scaler.cur_scale,
            "steps": model.global_steps, "opt_steps": model.optimizer.step_count}


def test_fp16_training_skips_overflowing_steps_and_recovers():
    """Start with an absurd loss scale: the first steps overflow in fp16, are skipped (weights untouched) and halve
    the scale until gradients are finite; training then proceeds."""
    cfg = tiny_config(use_cpu_initialization=True, precision="fp16",
                      fp16={"enabled": True, "loss_scale": 0, "initial_scale_power": 26, "loss_scale_window": 1000,
                            "hysteresis": 1, "min_loss_scale": 1})
    r = run_distributed(_train, 1, cfg, 24)[0]
    assert r["skipped"] >= 3 and r["skipped"] < 24
    assert r["scale"] == 2.0 ** 26 / 2 ** r["skipped"]
    assert all(l == l for l in r["losses"])
    assert r["losses"][-1] < r["losses"][0]
    # a skipped step is not an optimizer step: Adam's bias corrections count real updates only
    assert r["opt_steps"] == r["steps"] - r["skipped"]


def _train_hidden_gpu(rank, world, cfg, steps):
    """The same run with every GPU hidden from the child: the fp32 PyTorch oracle."""
    import os
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    return _train(rank, world, cfg, steps)


@pytest.mark.gpu
def test_fp16_trains_on_the_gpu_kernels_with_dynamic_loss_scaling():
    """precision fp16 on a B200: the fp16 builds of the kernels train the model; the loss curve follows the fp32
    PyTorch oracle (same seed, same CPU-side initialisation, same synthetic batches).  A second run starts from
    an absurd loss scale: the scaler sees the overflow through the device-side non-finite check, skips those
    steps, halves the scale each time and then trains (Adam with lr 2e-3 moves the weights enough in 16 steps for
    a wrong gradient to show in the curve)."""
    base = dict(use_cpu_initialization=True, num_layers=2, hidden_size=256, num_attention_heads=4, seq_length=256,
                max_position_embeddings=256, synthetic_vocab_size=1000, attention_config=[[["flash"], 2]],
                train_micro_batch_size_per_gpu=2, gradient_accumulation_steps=2,
                optimizer={"type": "Adam", "params": {"lr": 2e-3, "betas": [0.9, 0.95], "eps": 1e-8}})
    oracle = run_distributed(_train_hidden_gpu, 1, tiny_config(precision="fp32", **base), 16)[0]
    fp16 = dict(enabled=True, loss_scale=0, initial_scale_power=12, loss_scale_window=1000, hysteresis=1,
                min_loss_scale=1)
    r = run_distributed(_train, 1, tiny_config(precision="fp16", fp16=fp16, distributed_backend="nccl", **base), 16)[0]
    assert r["skipped"] == 0 and r["scale"] == 2.0 ** 12
    assert r["losses"] == pytest.approx(oracle["losses"], rel=2e-2), (r["losses"], oracle["losses"])
    huge = dict(fp16, initial_scale_power=26)
    r = run_distributed(_train, 1, tiny_config(precision="fp16", fp16=huge, distributed_backend="nccl", **base), 24)[0]
    assert 3 <= r["skipped"] < 24
    assert r["scale"] == 2.0 ** 26 / 2 ** r["skipped"]
    assert r["opt_steps"] == r["steps"] - r["skipped"]
    # while the steps are skipped the weights do not move: the loss stays at its initial value up to batch noise
    assert abs(r["losses"][1] - oracle["losses"][0]) < 0.2
    # uniform random tokens cannot be learned beyond their unigram statistics: after the skipped steps the run sits
    # at the oracle's level, with finite losses throughout
    assert all(l == l for l in r["losses"]) and abs(r["losses"][-1] - oracle["losses"][-1]) < 0.15
