"""muP: base shapes, width multipliers, init / learning-rate rules, read-out scaling, end-to-end training with a
saved base-shapes file, and the coordinate check (reference: megatron/training.py:73-170, mup package semantics)."""
import json
import os

import pytest
import torch

from common import run_distributed, tiny_config
from gpt_neox_b200 import mup


class _Net(torch.nn.Module):
    def __init__(self, width, vocab=11):
        super().__init__()
        self.emb = torch.nn.Embedding(vocab, width)
        self.fc = torch.nn.Linear(width, 4 * width)
        self.out = torch.nn.Linear(4 * width, width, bias=False)
        self.norm = torch.nn.LayerNorm(width)
        self.fixed = torch.nn.Linear(7, 3)


def test_base_shapes_infinite_dimensions_and_width_mult(tmp_path):
    base, delta, target = _Net(8), _Net(16), _Net(32)
    f = str(tmp_path / "shapes.0")
    shapes = mup.make_base_shapes(mup.get_shapes(base), mup.get_shapes(delta), savefile=f)
    assert shapes["emb.weight"] == [None, 8] and shapes["fc.weight"] == [32, 8] and shapes["fixed.weight"] == [None, None]
    mup.set_base_shapes(target, f)                                   # from the saved file
    assert target.emb.weight.infshape.ninf() == 1 and target.emb.weight.infshape.width_mult() == 4.0
    assert target.fc.weight.infshape.ninf() == 2 and target.fc.weight.infshape.width_mult() == 4.0   # fan-in 32 / 8
    assert target.fc.weight.infshape.fanin_fanout_mult_ratio() == 1.0
    assert target.fc.bias.infshape.ninf() == 1 and target.norm.weight.infshape.width_mult() == 4.0
    assert target.fixed.weight.infshape.ninf() == 0 and target.fixed.weight.infshape.width_mult() == 1.0
    with pytest.raises(FileNotFoundError):
        mup.load_base_shapes(str(tmp_path / "missing"))
    with pytest.raises(KeyError):
        mup.set_base_shapes(target, {"emb.weight": [None, 8]})


def test_apply_mup_rescales_matrix_like_weights_and_sets_multipliers():
    base, delta, target = _Net(8), _Net(16), _Net(32)
    shapes = mup.make_base_shapes(mup.get_shapes(base), mup.get_shapes(delta))
    mup.set_base_shapes(target, shapes)
    before = {n: p.detach().clone() for n, p in target.named_parameters()}
    mup.apply_mup(target, optimizer="adam")
    torch.testing.assert_close(target.fc.weight, before["fc.weight"] * 4.0 ** -0.5)       # std / sqrt(width_mult)
    torch.testing.assert_close(target.emb.weight, before["emb.weight"])                   # vector-like: unchanged
    torch.testing.assert_close(target.fixed.weight, before["fixed.weight"])
    assert target.fc.weight.lr_mult == 0.25 and target.fc.weight.wd_mult == 4.0
    assert target.emb.weight.lr_mult == 1.0 and target.fc.bias.lr_mult == 1.0 and target.fixed.weight.lr_mult == 1.0
    mup.apply_mup(target, optimizer="sgd", reinit=False)
    assert target.fc.weight.lr_mult == 1.0                   # fan-in and fan-out grow alike
    assert target.emb.weight.lr_mult == 4.0 and target.fixed.weight.lr_mult == 1.0
    with pytest.raises(ValueError):
        mup.lr_multiplier(target.fc.weight.infshape, "lion")


def test_engine_applies_per_parameter_lr_multiplier():
    """One Adam step moves every element by ~lr * sign(g): a parameter with lr_mult 0.25 moves a quarter as far."""
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.engine import engine as E
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(tiny_config(weight_decay=0.0, gradient_clipping=0.0))
    a.configure_distributed_args()
    from gpt_neox_b200.initialize import initialize_megatron
    initialize_megatron(a)
    torch.manual_seed(0)
    lin = torch.nn.Linear(6, 5)
    lin.weight.lr_mult = 0.25
    w0, b0 = lin.weight.detach().clone(), lin.bias.detach().clone()
    eng = E.Engine(lin, a, [{"params": list(lin.parameters()), "weight_decay": 0.0}],
                   optimizer_cfg={"lr": 0.1, "betas": (0.9, 0.999), "eps": 1e-12, "weight_decay": 0.0,
                                  "adam_w_mode": True})
    x = torch.randn(3, 6)
    eng.backward(lin(x).pow(2).sum())
    eng.step()
    dw, db = (lin.weight.detach() - w0).abs(), (lin.bias.detach() - b0).abs()
    torch.testing.assert_close(dw, torch.full_like(dw, 0.025), rtol=1e-3, atol=1e-6)
    torch.testing.assert_close(db, torch.full_like(db, 0.1), rtol=1e-3, atol=1e-6)
    mpu.destroy_model_parallel()


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
    try:
        training.pretrain(a)
    except SystemExit as e:
        return {"exit": e.code}
    return {"losses": losses}


def test_mup_training_end_to_end_with_saved_base_shapes(tmp_path):
    """`save_base_shapes` writes <file>.<rank> and stops; a 2x wider model then trains under muP with it, and at
    base width muP changes nothing but the attention scale (1/d instead of 1/sqrt(d))."""
    shapes = str(tmp_path / "base_shapes")
    base = tiny_config(use_cpu_initialization=True, use_mup=True, base_shapes_file=shapes, no_weight_tying=False)
    r = run_distributed(_train, 1, dict(base, save_base_shapes=True), 2)[0]
    assert r == {"exit": 1} and os.path.exists(shapes + ".0")
    import yaml
    with open(shapes + ".0") as f:
        saved = yaml.safe_load(f)
    assert any(v == [64 * 3, 64] or v == [192, 64] for v in saved.values())          # QKV: both dimensions grow
    same = run_distributed(_train, 1, base, 4)[0]["losses"]
    plain = run_distributed(_train, 1, dict(base, use_mup=False), 4)[0]["losses"]
    # width_mult == 1 everywhere: same init, learning rates and read-out; only the 1/d attention scale differs
    assert same[0] == pytest.approx(plain[0], rel=1e-4) and same == pytest.approx(plain, rel=5e-3)
    wide = run_distributed(_train, 1, dict(base, hidden_size=128), 6)[0]["losses"]
    assert len(wide) == 6 and all(l == l for l in wide) and wide[-1] < wide[0]
    wide_plain = run_distributed(_train, 1, dict(base, hidden_size=128, use_mup=False), 6)[0]["losses"]
    assert wide != pytest.approx(wide_plain, rel=1e-3)                               # muP changed init / lr / read-out


def _coord(rank, world, cfg, cwd):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world))
    a.configure_distributed_args()
    a.build_tokenizer()
    os.chdir(cwd)
    training.pretrain(a)
    return True


def test_coord_check_writes_activation_scales_per_width(tmp_path):
    shapes = str(tmp_path / "base_shapes")
    base = tiny_config(use_cpu_initialization=True, use_mup=True, base_shapes_file=shapes, num_attention_heads=2,
                       hidden_size=16, train_iters=1)
    run_distributed(_train, 1, dict(base, save_base_shapes=True), 1)
    cfg = dict(base, coord_check=True, mup_coord_check_widths=[16, 32, 64], mup_coord_check_steps=2)
    run_distributed(_coord, 1, cfg, str(tmp_path))
    for tag in ("up", "sp"):
        with open(tmp_path / f"coord_check_{tag}.0.json") as f:
            recs = json.load(f)
        assert {r["width"] for r in recs} == {16, 32, 64} and {r["t"] for r in recs} == {1, 2}
        assert all(r["l1"] >= 0 for r in recs)
        exps = mup.growth_exponents(recs)
        assert exps and all(abs(v) < 3 for v in exps.values())
