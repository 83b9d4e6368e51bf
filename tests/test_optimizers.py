"""SM3 / MADGRAD-WD / Lion: closed-form single steps and a convex problem (reference: megatron/optimizers.py)."""
import pytest
import torch

from gpt_neox_b200.optimizers import SM3, Lion, madgrad_wd


def _quad(opt_cls, steps=200, **kw):
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(6, 5))
    tgt = torch.randn(6, 5)
    opt = opt_cls([w], **kw)
    first = None
    for _ in range(steps):
        opt.zero_grad()
        loss = ((w - tgt) ** 2).sum()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    return first, loss.item()


@pytest.mark.parametrize("cls,kw", [(SM3, dict(lr=0.1)), (SM3, dict(lr=0.1, momentum=0.9, beta=0.5)),
                                    (madgrad_wd, dict(lr=0.05)), (madgrad_wd, dict(lr=0.05, momentum=0.0)),
                                    (Lion, dict(lr=0.01))])
def test_optimizers_minimise_a_quadratic(cls, kw):
    first, last = _quad(cls, **kw)
    assert last < 0.05 * first


def test_lion_single_step_closed_form():
    w = torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    w.grad = torch.tensor([0.5, -0.5, 0.0])
    Lion([w], lr=0.1, betas=(0.9, 0.99), weight_decay=0.1).step()
    exp = torch.tensor([1.0, -2.0, 3.0]) * (1 - 0.01) - 0.1 * torch.tensor([1.0, -1.0, 0.0])
    torch.testing.assert_close(w.data, exp)


def test_sm3_first_step_is_sign_like_and_covers_are_row_col_max():
    w = torch.nn.Parameter(torch.zeros(2, 3))
    g = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    w.grad = g.clone()
    opt = SM3([w], lr=1.0)
    opt.step()
    torch.testing.assert_close(w.data, -torch.ones(2, 3))          # g / sqrt(g^2)
    rows, cols = opt.state[w]["covers"]
    torch.testing.assert_close(rows.flatten(), torch.tensor([9.0, 36.0]))
    torch.testing.assert_close(cols.flatten(), torch.tensor([16.0, 25.0, 36.0]))


def test_madgrad_first_step_closed_form():
    w = torch.nn.Parameter(torch.tensor([1.0, 2.0]))
    g = torch.tensor([0.5, -1.0])
    w.grad = g.clone()
    lr, eps, mom = 0.1, 1e-6, 0.9
    madgrad_wd([w], lr=lr, momentum=mom, eps=eps).step()
    lam = (lr + eps) * 1.0
    z = torch.tensor([1.0, 2.0]) - lam * g / ((lam * g * g).pow(1 / 3) + eps)
    exp = torch.tensor([1.0, 2.0]) * mom + (1 - mom) * z
    torch.testing.assert_close(w.data, exp)


@pytest.mark.parametrize("name,params", [("sm3", {"lr": 0.01}), ("lion", {"lr": 1e-4, "betas": [0.9, 0.99]}),
                                          ("madgrad_wd", {"lr": 0.01, "momentum": 0.9}), ("sgd", {"lr": 0.01})])
def test_engine_runs_with_in_tree_optimizers(name, params):
    from common import run_distributed, tiny_config
    from test_mamba import _train
    cfg = tiny_config(use_cpu_initialization=True, optimizer={"type": name, "params": params})
    losses = run_distributed(_train, 1, cfg, 4)[0]
    assert all(l == l for l in losses)


def _losses_with(rank, world, cfg, steps):
    import torch
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world, train_iters=steps, lr_decay_iters=steps))
    a.configure_distributed_args()
    a.build_tokenizer()
    losses = []
    training.collect_loss_for_unit_test = lambda l: losses.append(float(l))
    model = training.pretrain(a)
    return losses, float(model.get_global_grad_norm())


def test_gradient_predivide_and_prescale_leave_the_step_unchanged():
    """``gradient_predivide_factor`` / ``prescale_gradients`` move the data-parallel average in front of the
    reduction and ``communication_data_type`` picks its dtype: in fp32 the losses and the reported gradient
    norm stay those of the default engine."""
    import pytest
    from common import run_distributed, tiny_config
    cfg = tiny_config(use_cpu_initialization=True)
    ref = run_distributed(_losses_with, 2, cfg, 4)[0]
    for over in (dict(gradient_predivide_factor=2.0), dict(prescale_gradients=True),
                 dict(gradient_predivide_factor=4.0, communication_data_type="fp32"),
                 dict(zero_optimization={"stage": 0}, prescale_gradients=True)):
        got = run_distributed(_losses_with, 2, dict(cfg, **over), 4)[0]
        if "zero_optimization" in over:
            base = run_distributed(_losses_with, 2, dict(cfg, zero_optimization={"stage": 0}), 4)[0]
        else:
            base = ref
        assert got[0] == pytest.approx(base[0], rel=1e-5), over
        assert got[1] == pytest.approx(base[1], rel=1e-4), over


def test_8bit_adam_state_codes_round_trip_within_a_few_percent():
    from gpt_neox_b200.ops.optim import q8_blocks, q8_decode, q8_encode
    torch.manual_seed(0)
    n = 5000
    m = torch.randn(n) * torch.rand(n) ** 4
    v = torch.randn(n) ** 2 * 1e-3
    m8, v8, sm, sv = q8_encode(m, v)
    assert m8.dtype == torch.uint8 and sm.numel() == q8_blocks(n) == 3
    m2, v2 = q8_decode(m8, v8, sm, sv)
    big = m.abs() > 1e-3 * m.abs().max()
    assert ((m2 - m).abs() / m.abs())[big].max() < 0.045 and torch.equal(torch.sign(m2[big]), torch.sign(m[big]))
    assert ((v2 - v).abs() / v)[v > 1e-7 * v.max()].max() < 0.045
    z8, _, zs, _ = q8_encode(torch.zeros(10), torch.zeros(10))
    assert int(z8.sum()) == 0 and float(zs.sum()) == 0.0          # all-zero state is all-zero codes


def test_8bit_adam_follows_32bit_adam_in_the_engine():
    """``use_bnb_optimizer``: the engine keeps the Adam moments in 8 bits (ZeRO-1 over two ranks); the loss curve
    stays close to the fp32-state run, and the state really is one byte per element."""
    import pytest
    from common import run_distributed, tiny_config
    cfg = tiny_config(use_cpu_initialization=True, num_layers=2, hidden_size=128)
    ref = run_distributed(_losses_with, 2, cfg, 12)[0][0]
    got = run_distributed(_losses_with, 2, dict(cfg, use_bnb_optimizer=True), 12)[0][0]
    assert got[0] == pytest.approx(ref[0], rel=1e-6)
    assert got == pytest.approx(ref, rel=3e-2)
    assert got[-1] < got[0]


def _compressed_mean(rank, world, steps):
    import torch
    import torch.distributed as dist
    from gpt_neox_b200.optimizers import CompressedAllreduce
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(100 + rank)
    x = torch.randn(1000)                                   # this rank's (constant) vector
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x)
    mean = torch.stack(parts).mean(0)
    car = CompressedAllreduce(x.numel(), dist.group.WORLD, x.device)
    acc = torch.zeros_like(x)
    first = None
    for _ in range(steps):
        out = car(x.clone())
        first = out.clone() if first is None else first
        acc += out
    dist.destroy_process_group()
    one = ((first - mean).norm() / mean.norm()).item()
    avg = ((acc / steps - mean).norm() / mean.norm()).item()
    return one, avg, first.tolist()[:8]


def test_compressed_allreduce_is_unbiased_over_time_and_identical_on_all_ranks():
    """One call gives a 1-bit approximation of the mean (large error); with error feedback on both stages the
    time average of repeated calls converges to the true mean; every rank ends up with the same vector."""
    from common import run_distributed
    out = run_distributed(_compressed_mean, 2, 64)
    (one0, avg0, head0), (one1, avg1, head1) = out
    assert head0 == head1
    assert one0 > 0.3 and avg0 < 0.1 and avg0 < one0 / 4, (one0, avg0)


def _onebit_run(rank, world, cfg, steps):
    import torch
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world, train_iters=steps, lr_decay_iters=steps))
    a.configure_distributed_args()
    a.build_tokenizer()
    losses = []
    training.collect_loss_for_unit_test = lambda l: losses.append(float(l))
    model = training.pretrain(a)
    opt = model.optimizer.generic
    checksum = float(sum(p.double().sum() for p in model.module.parameters()))
    return losses, opt.steps, opt.compression_steps, checksum


def test_onebit_adam_trains_with_compressed_momentum_after_the_warmup():
    """OneBitAdam on two data-parallel ranks (gloo): plain Adam on reduced gradients for ``freeze_step`` steps, then
    local gradients + the 1-bit momentum all-reduce.  The loss keeps falling in the compressed phase and the
    replicas stay bit-identical (same parameter checksum on both ranks)."""
    from common import run_distributed, tiny_config
    cfg = tiny_config(use_cpu_initialization=True, zero_optimization={"stage": 0}, num_layers=2, hidden_size=128,
                      optimizer={"type": "OneBitAdam", "params": {"lr": 1e-3, "freeze_step": 6, "betas": [0.9, 0.95]}})
    (l0, steps, comp, c0), (l1, _, _, c1) = run_distributed(_onebit_run, 2, cfg, 16)
    assert (steps, comp) == (16, 10)
    assert c0 == c1
    assert min(l0[6:]) < l0[5] and l0[-1] < l0[0]
    assert all(x == x for x in l0)


@pytest.mark.parametrize("over", [dict(optimizer={"type": "cpu_adam", "params": {"lr": 6e-4, "betas": [0.9, 0.95], "eps": 1e-8}}),
                                  dict(optimizer={"type": "cpu_torch_adam", "params": {"lr": 6e-4, "betas": [0.9, 0.95], "eps": 1e-8}}),
                                  dict(zero_optimization={"stage": 3, "offload_optimizer": {"device": "cpu"}})],
                         ids=["cpu_adam", "cpu_torch_adam", "zero3_offload_optimizer"])
def test_optimizer_state_offload_matches_the_device_optimizer(over):
    """Master weights and Adam moments held on the host (native multi-threaded AdamW, or PyTorch's CPU operators for
    ``cpu_torch_adam``), two data-parallel ranks: the loss curve is that of the in-place optimizer."""
    from common import run_distributed, tiny_config
    cfg = tiny_config(use_cpu_initialization=True)
    ref = run_distributed(_losses_with, 2, cfg, 6)[0]
    got = run_distributed(_losses_with, 2, dict(cfg, **over), 6)[0]
    assert got[0] == pytest.approx(ref[0], rel=2e-5)
    assert got[1] == pytest.approx(ref[1], rel=1e-4)


def test_native_host_adamw_matches_the_torch_statement_for_every_dtype_pair():
    from gpt_neox_b200.ops.optim import adamw_step_, cpu_adamw_step_
    torch.manual_seed(0)
    for gd, lpd in ((torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                    (torch.float32, torch.float32)):
        n = 70001
        p, m, v = torch.randn(n), torch.zeros(n), torch.zeros(n)
        lp = torch.empty(n, dtype=lpd)
        p2, m2, v2, lp2 = p.clone(), m.clone(), v.clone(), lp.clone()
        for step in range(1, 4):
            g = torch.randn(n).to(gd)
            kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
            cpu_adamw_step_(p, m, v, g, lp, grad_scale=0.5, **kw)
            adamw_step_(p2, m2, v2, g, lp2, grad_scale=torch.tensor([0.5]), **kw)
        torch.testing.assert_close(p, p2, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(v, v2, rtol=1e-5, atol=1e-7)
        assert (lp.float() - lp2.float()).abs().max() <= 2.0 ** -7 * lp2.float().abs().max()
