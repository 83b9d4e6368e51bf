"""Post-training objectives (reward model, DPO, KTO, REINFORCE): closed-form values of the loss functions and the
``forward_step`` wiring of every ``train_impl`` on a tiny CPU model (reference: megatron/training.py:600-859)."""
import copy
import math

import pytest
import torch
import torch.nn.functional as F

from common import tiny_config


@pytest.fixture(scope="module", autouse=True)
def _single_rank():
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(tiny_config())
    a.configure_distributed_args()
    a.build_tokenizer()
    initialize_megatron(a)
    yield
    mpu.destroy_model_parallel()


def _logp_ref(logits, labels):
    return torch.gather(torch.log_softmax(logits.float(), -1), 2, labels.unsqueeze(-1)).squeeze(-1)


def test_get_logp_is_the_label_log_probability():
    from gpt_neox_b200 import posttrain
    torch.manual_seed(0)
    logits, labels = torch.randn(4, 6, 11), torch.randint(0, 11, (4, 6))
    torch.testing.assert_close(posttrain.get_logp(logits, labels), _logp_ref(logits, labels), rtol=1e-5, atol=1e-5)
    pos, neg = posttrain.get_pos_neg_logp(logits, labels)
    torch.testing.assert_close(torch.cat((pos, neg)), _logp_ref(logits, labels), rtol=1e-5, atol=1e-5)


def test_dpo_loss_closed_form_and_metrics():
    from gpt_neox_b200 import posttrain
    torch.manual_seed(1)
    logits, labels = torch.randn(4, 5, 9, requires_grad=True), torch.randint(0, 9, (4, 5))
    mask = torch.ones(4, 5)
    mask[:, 0] = 0
    lp = (_logp_ref(logits.detach(), labels) * mask).sum(-1)
    ref_pos, ref_neg = torch.tensor([-7.0, -6.0]), torch.tensor([-6.5, -7.5])
    beta = 0.3
    loss, m = posttrain.dpo_loss(logits, labels, mask, ref_pos, ref_neg, beta, False, True)
    want = -F.logsigmoid(beta * ((lp[:2] - lp[2:]) - (ref_pos - ref_neg))).mean()
    torch.testing.assert_close(loss.detach(), want, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(m["margins"], (beta * ((lp[:2] - ref_pos) - (lp[2:] - ref_neg))).mean(), rtol=1e-5, atol=1e-6)
    loss.backward()
    assert logits.grad.abs().sum() > 0 and logits.grad[:, 0].abs().sum() == 0        # masked position: no gradient
    # policy == reference: the loss is log 2 whatever beta is
    same, _ = posttrain.dpo_loss(logits.detach(), labels, mask, lp[:2], lp[2:], 5.0, False, True)
    assert float(same) == pytest.approx(math.log(2.0), rel=1e-5)


def test_rm_loss_reads_the_last_unmasked_position():
    from gpt_neox_b200 import posttrain
    values = torch.tensor([[[0.0], [2.0], [9.0]], [[0.0], [0.0], [1.0]],          # chosen
                           [[0.0], [0.5], [9.0]], [[0.0], [0.0], [3.0]]])         # rejected
    mask = torch.tensor([[0, 1, 0], [0, 0, 1], [0, 1, 0], [0, 0, 1]], dtype=torch.float32)
    loss, m = posttrain.rm_loss(values, mask, z_loss=0.0)
    pos, neg = torch.tensor([2.0, 1.0]), torch.tensor([0.5, 3.0])
    assert float(loss) == pytest.approx(float(-F.logsigmoid(pos - neg).mean()), rel=1e-6)
    assert float(m["accuracy"]) == 0.5 and float(m["margin"]) == pytest.approx(-0.25)
    # a whole completion labelled: still the last unmasked position of each row
    wide = torch.tensor([[1, 1, 0], [0, 1, 1], [1, 1, 0], [1, 1, 1]], dtype=torch.float32)
    same, _ = posttrain.rm_loss(values, wide, z_loss=0.0)
    assert float(same) == pytest.approx(float(loss))
    with_z, _ = posttrain.rm_loss(values, mask, z_loss=0.1)
    assert float(with_z - loss) == pytest.approx(0.1 * float((pos ** 2 + neg ** 2).mean()), rel=1e-6)


def test_kto_loss_equal_policy_and_reference_and_sign_of_the_push():
    from gpt_neox_b200 import posttrain
    logp = torch.full((4, 3), -1.0)
    mask = torch.ones(4, 3)
    rewards = torch.tensor([[1.0] * 3, [-1.0] * 3, [1.0] * 3, [-1.0] * 3])
    loss, m = posttrain.kto_loss(logp, logp.clone(), rewards, mask, beta=0.1, desirable_weight=1.0, undesirable_weight=1.0)
    assert float(loss) == pytest.approx(0.5)                         # 2 halves x 0.5 x (1 - sigmoid(0))
    assert float(m["kl"]) == 0.0
    # raising the log-probability of a desirable sample lowers the loss; of an undesirable one raises it
    up_good = logp.clone(); up_good[0] += 1.0
    up_bad = logp.clone(); up_bad[1] += 1.0
    l_good, _ = posttrain.kto_loss(up_good, logp, rewards, mask, 0.1, 1.0, 1.0)
    l_bad, _ = posttrain.kto_loss(up_bad, logp, rewards, mask, 0.1, 1.0, 1.0)
    assert float(l_good) < 0.5 < float(l_bad)
    # the weights scale their own class only
    l_w, _ = posttrain.kto_loss(up_bad, logp, rewards, mask, 0.1, 1.0, 2.0)
    assert float(l_w) > float(l_bad)


@pytest.mark.parametrize("kl_impl", ["abs", "mse", "kl", "full"])
def test_reinforce_loss_matches_the_statement(kl_impl):
    from gpt_neox_b200 import posttrain
    torch.manual_seed(2)
    logits, ref_logits = torch.randn(3, 4, 7), torch.randn(3, 4, 7)
    labels = torch.randint(0, 7, (3, 4))
    mask = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]], dtype=torch.float32)
    rewards = torch.tensor([[0.5], [-1.0], [2.0]]).expand(3, 4).contiguous()
    raw = torch.tensor([1.0, 0.0, 3.0])
    lp, rlp = _logp_ref(logits, labels), _logp_ref(ref_logits, labels)
    plain, m0 = posttrain.reinforce_loss(logits, None, labels, mask, rewards, raw, kl_impl, 0.0, True)
    want = ((-(rewards * lp) * mask).sum(-1) / mask.sum()).mean()
    torch.testing.assert_close(plain, want, rtol=1e-5, atol=1e-6)
    assert float(m0["reward"]) == pytest.approx(float(raw.mean()))
    beta = 0.2
    got, m = posttrain.reinforce_loss(logits, ref_logits, labels, mask, rewards, raw, kl_impl, beta, True)
    d = lp - rlp
    if kl_impl == "full":
        a, b = torch.log_softmax(logits, -1), torch.log_softmax(ref_logits, -1)
        kl = (a.exp() * (a - b)).sum(-1)
    else:
        kl = {"abs": d.abs(), "mse": 0.5 * d * d, "kl": d}[kl_impl]
    want = (((-(rewards * lp) + beta * kl) * mask).sum(-1) / mask.sum()).mean()
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    assert float(m["kl"]) == pytest.approx(float(kl.mean()), rel=1e-4, abs=1e-5)


# ------------------------------------------------------------------------------------------ forward_step wiring
def _model(**over):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(tiny_config(use_cpu_initialization=True, train_micro_batch_size_per_gpu=2, **over))
    a.configure_distributed_args()
    a.build_tokenizer()
    initialize_megatron(a)
    torch.manual_seed(3)
    return a, training.get_model(a)


def _pairs(n=2, s=33, vocab=100, seed=4):
    g = torch.Generator().manual_seed(seed)
    tok = lambda: torch.randint(1, vocab, (n, s), generator=g)
    pos, neg = tok(), tok()
    lab = lambda t: torch.where(torch.arange(s)[None] >= 8, t, torch.full_like(t, -100))   # prompt masked out
    return {"pos": pos, "neg": neg, "pos_label": lab(pos), "neg_label": lab(neg)}


def test_forward_step_dpo_starts_at_log2_and_learns():
    from gpt_neox_b200 import training
    a, model = _model(train_impl="dpo", dpo_beta=0.5, dpo_fp32=True, pos_train_label_data_paths=["x"],
                      neg_train_label_data_paths=["x"], pos_train_data_paths=["x"], neg_train_data_paths=["x"])
    ref = copy.deepcopy(model)
    batch = _pairs()
    loss, metrics = training.forward_step(iter([batch]), model, a, None, is_train=True, reference_model=ref)
    assert loss.item() == pytest.approx(math.log(2.0), rel=1e-4)
    assert float(metrics["margins"]) == pytest.approx(0.0, abs=1e-5)
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    for _ in range(8):
        opt.zero_grad()
        loss, metrics = training.forward_step(iter([batch]), model, a, None, is_train=True, reference_model=ref)
        loss.backward()
        opt.step()
    assert loss.item() < math.log(2.0) - 0.05 and float(metrics["reward_acc"]) == 1.0


def test_forward_step_reward_model_uses_a_scalar_head():
    from gpt_neox_b200 import training
    a, model = _model(train_impl="rm", z_loss=0.0, pos_train_label_data_paths=["x"], neg_train_label_data_paths=["x"],
                      pos_train_data_paths=["x"], neg_train_data_paths=["x"])
    batch = _pairs()
    for k in ("pos_label", "neg_label"):              # reward models score one position: the last token
        lab = torch.full_like(batch[k], -100)
        lab[:, -1] = batch[k[:3]][:, -1]
        batch[k] = lab
    loss, outputs, metrics = training.forward_step(iter([batch]), model, a, None, return_logits=True, is_train=True)
    assert outputs.shape[-1] == 1 and outputs.shape[0] == 4
    assert torch.isfinite(loss) and 0.0 <= float(metrics["accuracy"]) <= 1.0
    loss.backward()
    assert sum(float(p.grad.abs().sum()) for p in model.parameters() if p.grad is not None) > 0


def test_forward_step_kto_and_reinforce():
    from gpt_neox_b200 import training
    a, model = _model(train_impl="kto", kto_beta=0.1, kto_fp32=True, train_label_data_paths=["x"], train_data_paths=["x"],
                      valid_data_paths=["x"], test_data_paths=["x"])
    ref = copy.deepcopy(model)
    g = torch.Generator().manual_seed(5)
    text = torch.randint(1, 100, (2, 33), generator=g)
    label = torch.where(torch.arange(33)[None] >= 8, text, torch.full_like(text, -100))
    reward = torch.tensor([[1.0], [-1.0]]).expand(2, 33).contiguous()
    loss, metrics = training.forward_step(iter([{"text": text, "label": label, "reward": reward}]), model, a, None,
                                          is_train=True, reference_model=ref)
    assert float(loss) == pytest.approx(0.5, rel=1e-5) and float(metrics["kl"]) == pytest.approx(0.0, abs=1e-6)

    a, model = _model(train_impl="reinforce", kl_div_beta=0.0, fp32_reinforce=True, train_label_data_paths=["x"],
                      train_data_paths=["x"], valid_data_paths=["x"], test_data_paths=["x"])
    rw = torch.tensor([[0.7], [-0.3]]).expand(2, 32).contiguous()
    raw = torch.tensor([1.0, 0.0])
    loss, metrics = training.forward_step(
        iter([{"text": text, "label": label, "reward": rw, "raw_reward": raw}]), model, a, None, is_train=True)
    assert torch.isfinite(loss) and float(metrics["reward"]) == pytest.approx(0.5)
    loss.backward()
