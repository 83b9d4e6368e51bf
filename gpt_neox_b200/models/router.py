"""MoE routers (megatron/model/router.py:24-275): top-k token choice (softmax -> top-k, optional
input jitter) and Sinkhorn (balanced assignment from 3 Sinkhorn iterations during training,
sigmoid / softmax scores).  Every rank computes its routing locally and deterministically: there is
no "rank 0 routes and broadcasts" step as in the reference (router.py:130-186), because ranks of one
expert-parallel group route different tokens."""
from __future__ import annotations

import torch
import torch.nn as nn


def _device(neox_args):
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and \
        not getattr(neox_args, "use_cpu_initialization", False) else torch.device("cpu")


class TopKTokenChoiceRouter(nn.Module):
    def __init__(self, neox_args, init_method):
        super().__init__()
        self.jitter_eps = neox_args.moe_jitter_eps
        self.top_k = neox_args.moe_top_k
        self.layer = nn.Linear(neox_args.hidden_size, neox_args.moe_num_experts, bias=False,
                               dtype=neox_args.params_dtype, device=_device(neox_args))
        init_method(self.layer.weight)

    def jitter(self, x):
        low, high = 1.0 - self.jitter_eps, 1.0 + self.jitter_eps
        return low + torch.rand(x.size(), dtype=x.dtype, device=x.device) * (high - low)

    def _top_k(self, scores):
        if self.top_k == 1:
            return scores.max(dim=-1, keepdim=True)
        return torch.topk(scores, self.top_k, dim=-1)

    def forward(self, x):
        """x [s, b, h] -> (expert_weights [s*b, k], expert_indices [s*b, k])."""
        if self.training and self.jitter_eps is not None:
            x = x * self.jitter(x)
        logits = torch.nn.functional.linear(x.reshape(-1, x.shape[-1]), self.layer.weight)
        scores = logits.float().softmax(dim=-1).to(x.dtype)
        return self._top_k(scores)


class SinkhornRouter(nn.Module):
    def __init__(self, neox_args, init_method):
        super().__init__()
        self.top_k = neox_args.moe_top_k
        self.params_dtype = neox_args.params_dtype
        self.layer = nn.Linear(neox_args.hidden_size, neox_args.moe_num_experts, bias=False,
                               dtype=neox_args.params_dtype, device=_device(neox_args))
        init_method(self.layer.weight)

    @staticmethod
    def sinkhorn(cost, tol=0.0001, max_iter=3):
        cost = torch.exp(cost)
        d0 = torch.ones(cost.size(0), device=cost.device, dtype=cost.dtype)
        d1 = 1 / (cost.size(1) * torch.sum(cost, 0))
        eps = 0.00000001
        d1_old = d1
        for _ in range(max_iter):
            d0 = (1 / d0.size(0)) * 1 / (torch.sum(d1 * cost, 1) + eps)
            d1 = (1 / d1.size(0)) * 1 / (torch.sum(d0.unsqueeze(1) * cost, 0) + eps)
            error = torch.mean(torch.abs(d1_old - d1))
            d1_old = d1
            if error < tol:
                break
        return d1 * cost * d0.unsqueeze(1)

    def _activation(self, logits):
        if self.top_k == 1:
            return torch.sigmoid(logits)
        return torch.softmax(logits, dim=-1, dtype=torch.float32).type_as(logits)

    def sinkhorn_load_balancing(self, logits):
        if self.training:
            with torch.no_grad():
                norm_logits = self.sinkhorn(logits.to(dtype=torch.float32))
                _, indices = torch.topk(norm_logits, k=self.top_k, dim=1)
            scores = torch.gather(self._activation(logits), 1, indices)
        else:
            scores, indices = torch.topk(self._activation(logits), k=self.top_k, dim=1)
        return scores, indices

    def forward(self, x):
        logits = torch.nn.functional.linear(x.reshape(-1, x.shape[-1]), self.layer.weight)
        return self.sinkhorn_load_balancing(logits)
