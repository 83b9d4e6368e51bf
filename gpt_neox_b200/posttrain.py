"""Post-training objectives: reward modelling, DPO, KTO and REINFORCE
(inline in the reference's ``forward_step``, megatron/training.py:600-859).

Per-token log-probabilities come from the vocab-parallel cross-entropy kernel
(``logp = -CE(logits, label)``), so no rank ever materialises the full-vocabulary softmax unless
``kl_impl == "full"`` asks for it.  ``get_pos_neg_logp`` is defined here; the reference calls it but
never defines it (megatron/training.py:644,659).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import parallel as mpu
from .parallel.mappings import gather_from_model_parallel_region


def get_logp(logits, labels, force_fp32=False):
    """Per-token log-probability of ``labels`` under vocab-parallel ``logits`` [b, s, V/p]."""
    if force_fp32:
        logits = logits.float()
    safe = labels.clone()
    safe[safe < 0] = 0
    return -mpu.vocab_parallel_cross_entropy(logits.contiguous(), safe)


def get_pos_neg_logp(logits, labels, force_fp32=False):
    """Log-probabilities of the chosen (first half of the batch) and rejected (second half)."""
    logp = get_logp(logits, labels, force_fp32)
    return torch.chunk(logp, 2, 0)


def _first(x):
    return x[0] if isinstance(x, tuple) else x


def rm_loss(outputs, loss_mask, z_loss):
    """Bradley-Terry loss on the scalar head at the last unmasked position of each sequence."""
    metrics = {}
    pos, neg = torch.chunk(_first(outputs), 2, 0)
    pos_mask, neg_mask = torch.chunk(loss_mask, 2, 0)
    # the score of a sequence is read at its LAST unmasked position (data prepared for reward modelling labels
    # only that token; with a whole completion labelled the last of its tokens is taken)
    last = lambda m: (m > 0).float().mul(torch.arange(1, m.shape[1] + 1, device=m.device)).argmax(dim=1, keepdim=True)
    pos_idx, neg_idx = last(pos_mask), last(neg_mask)
    pos = torch.gather(pos.squeeze(-1), dim=1, index=pos_idx)
    neg = torch.gather(neg.squeeze(-1), dim=1, index=neg_idx)
    with torch.no_grad():
        metrics["pos_values"] = pos.detach().mean()
        metrics["neg_values"] = neg.detach().mean()
        metrics["margin"] = (pos - neg).detach().mean()
        metrics["accuracy"] = ((pos - neg) > 0).detach().float().mean()
    loss = (-F.logsigmoid(pos - neg).mean()) + ((z_loss * (pos ** 2 + neg ** 2)).mean())
    return loss, metrics


def dpo_loss(model_outputs, labels, loss_mask, ref_pos, ref_neg, beta, reference_free, fp32):
    """``-log sigmoid(beta * ((pi_pos - pi_neg) - (ref_pos - ref_neg)))`` on sequence log-probs."""
    metrics = {}
    pos_mask, neg_mask = torch.chunk(loss_mask, 2, 0)
    chosen_pos, chosen_neg = get_pos_neg_logp(_first(model_outputs), labels, fp32)
    chosen_pos = (chosen_pos * pos_mask).sum(-1)
    chosen_neg = (chosen_neg * neg_mask).sum(-1)
    with torch.no_grad():
        if not reference_free:
            metrics["ref_neg"] = ref_neg.detach().mean()
            metrics["ref_pos"] = ref_pos.detach().mean()
        metrics["chosen_neg"] = chosen_neg.detach().mean()
        metrics["chosen_pos"] = chosen_pos.detach().mean()
        if not reference_free:
            cr = beta * (chosen_pos.detach() - ref_pos.detach())
            rr = beta * (chosen_neg.detach() - ref_neg.detach())
            metrics["chosen_rewards"] = cr.mean()
            metrics["rejected_rewards"] = rr.mean()
            metrics["reward_acc"] = (cr > rr).float().mean()
            metrics["margins"] = (cr - rr).mean()
    logits = (chosen_pos - chosen_neg) - (ref_pos - ref_neg)
    return -F.logsigmoid(beta * logits).mean(), metrics


def kto_loss(chosen_logp, ref_logp, rewards, loss_mask, beta, desirable_weight, undesirable_weight):
    """KTO with the KL baseline of each half of the batch estimated on the other half."""
    metrics = {}
    with torch.no_grad():
        ref_logp = ref_logp * loss_mask
        scaling = (rewards.sum(-1) > 0.001).float() * desirable_weight
        scaling = scaling + (rewards.sum(-1) < -0.001).float() * undesirable_weight
        pos_mask = (rewards > 0.001).float()
        neg_mask = (rewards < -0.001).float()
    chosen_logp = chosen_logp * loss_mask
    with torch.no_grad():
        metrics["ref_logp"] = ref_logp.sum(-1).mean()
        metrics["policy_logp"] = chosen_logp.detach().sum(-1).mean()
        metrics["pos_ref_logp"] = (ref_logp * pos_mask).sum(-1).mean()
        metrics["neg_ref_logp"] = (ref_logp * neg_mask).sum(-1).mean()
        metrics["pos_policy_logp"] = (chosen_logp.detach() * pos_mask).sum(-1).mean()
        metrics["neg_policy_logp"] = (chosen_logp.detach() * neg_mask).sum(-1).mean()
        metrics["kl"] = (chosen_logp.detach() - ref_logp).sum() / loss_mask.sum()
        policy_rewards = beta * rewards * (chosen_logp.detach() - ref_logp)
        metrics["reward_acc"] = (policy_rewards.sum(-1) > 0.0).float().mean()
        metrics["policy_rewards"] = policy_rewards.sum()
    p1, p2 = torch.chunk(chosen_logp, 2, 0)
    r1, r2 = torch.chunk(ref_logp, 2, 0)
    w1, w2 = torch.chunk(rewards, 2, 0)
    s1, s2 = torch.chunk(scaling, 2, 0)
    kl1 = torch.clamp((p1 - r1).sum(-1), min=0).mean()
    kl2 = torch.clamp((p2 - r2).sum(-1), min=0).mean()
    lr1, lr2 = p1 - r1, p2 - r2
    loss = (0.5 * s1.mean(-1) * (1 - torch.sigmoid(beta * w1.mean(-1) * (lr1.sum(-1) - kl2.detach())))) + \
           (0.5 * s2.mean(-1) * (1 - torch.sigmoid(beta * w2.mean(-1) * (lr2.sum(-1) - kl1.detach()))))
    return loss.mean(), metrics


def reinforce_loss(outputs, ref_outputs, labels, loss_mask, rewards, raw_rewards, kl_impl, kl_beta, fp32):
    """Policy gradient with an optional per-token KL penalty against a reference model
    (``kl_impl``: abs | mse | kl on sampled tokens, or ``full`` over the vocabulary)."""
    metrics = {}
    outputs = _first(outputs)
    ref_per_token = ref_logp_full = None
    if ref_outputs is not None:
        with torch.no_grad():
            ref_outputs = _first(ref_outputs)
            if kl_impl == "full":
                ro = gather_from_model_parallel_region(ref_outputs)
                ro = ro.float() if fp32 else ro
                ref_logp_full = ro.log_softmax(dim=-1).detach()
                ref_per_token = torch.gather(ref_logp_full, 2, labels.unsqueeze(2)).squeeze(2)
            else:
                ref_per_token = get_logp(ref_outputs, labels, fp32)
            metrics["ref_logp"] = ref_per_token.detach().mean()
    if kl_impl == "full":
        o = gather_from_model_parallel_region(outputs)
        o = o.float() if fp32 else o
        logp_full = o.log_softmax(dim=-1)
        per_token = torch.gather(logp_full, 2, labels.unsqueeze(2)).squeeze(2)
    else:
        logp_full = None
        per_token = get_logp(outputs, labels, fp32)
    with torch.no_grad():
        metrics["logp"] = per_token.detach().mean()
        metrics["reward"] = raw_rewards.detach().mean()
        metrics["reward_std"] = raw_rewards.detach().std()
    denom = loss_mask.sum()
    if ref_outputs is not None:
        if kl_impl == "full":
            kl = F.kl_div(ref_logp_full, logp_full, log_target=True, reduction="none").sum(-1)
        else:
            kl = per_token - ref_per_token
            if kl_impl == "abs":
                kl = kl.abs()
            elif kl_impl == "mse":
                kl = 0.5 * kl.square()
        with torch.no_grad():
            metrics["kl"] = kl.detach().mean()
        loss = (-per_token * rewards) + (kl_beta * kl)
    else:
        loss = -(rewards * per_token)
    loss = ((loss * loss_mask).sum(-1) / denom).mean()
    return loss, metrics
