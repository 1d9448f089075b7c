"""The routers PiKVMoE wires up, with the surface of core/single/routing_strategy.py.

Each ExpertRouter tail (temperature, additive mask, softmax, top-k, renormalisation) is one call of
the fused gate kernel on the gate net's hidden activations; the mixture of the two strategies and
its final top-k run on the kernel again (the mixed weights are probabilities, so their logarithm is
handed over as logits: softmax(log w) = w).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, ops


class ExpertRouter(nn.Module):
    """core/single/routing_strategy.py:6-55."""

    def __init__(self, hidden_size, num_experts, top_k=2, temperature=1.0):
        super().__init__()
        self.hidden_size, self.num_experts, self.top_k, self.temperature = hidden_size, num_experts, top_k, temperature
        self.router = nn.Sequential(nn.Linear(hidden_size, hidden_size), nn.ReLU(), nn.Linear(hidden_size, num_experts))
        self.expert_capacity = nn.Parameter(torch.ones(num_experts))
        self.last_gate = None

    def _gate(self, x, expert_mask=None):
        b, s, h = x.shape
        act = F.relu(self.router[0](x.reshape(-1, h)))
        last = self.router[2]
        g = ops.gate_fused(act, last.weight.detach().to(act.dtype), last.bias.detach(), top_k=self.top_k,
                           expert_mask=expert_mask, mask_mode=_lib.MASK_BIAS, temperature=self.temperature)
        self.last_gate = g
        return g

    def forward(self, x, expert_mask=None):
        b, s, _ = x.shape
        g = self._gate(x, expert_mask)
        return (g.probs.view(b, s, self.num_experts), g.topk_idx.view(b, s, self.top_k).long(),
                g.topk_w.view(b, s, self.top_k))


class LoadBalancingRouter(ExpertRouter):
    """core/single/routing_strategy.py:57-71."""

    def __init__(self, hidden_size, num_experts, top_k=2, temperature=1.0, balance_weight=0.01):
        super().__init__(hidden_size, num_experts, top_k, temperature)
        self.balance_weight = balance_weight

    def forward(self, x, expert_mask=None):
        w, idx, tw = super().forward(x, expert_mask)
        usage = self.last_gate.prob_sum / float(x.shape[0] * x.shape[1])
        return w, idx, tw, self.balance_weight * (usage.std() / usage.mean())


class ImportanceAwareRouter(ExpertRouter):
    """core/single/routing_strategy.py:73-98."""

    def __init__(self, hidden_size, num_experts, top_k=2, temperature=1.0):
        super().__init__(hidden_size, num_experts, top_k, temperature)
        self.importance_predictor = nn.Sequential(nn.Linear(hidden_size, hidden_size // 2), nn.ReLU(),
                                                  nn.Linear(hidden_size // 2, 1), nn.Sigmoid())

    def forward(self, x, expert_mask=None):
        importance = self.importance_predictor(x)
        w, idx, tw = super().forward(x, expert_mask)
        w = w * importance
        w = w / w.sum(dim=-1, keepdim=True)
        return w, idx, tw, importance


class AdaptiveRouter(nn.Module):
    """core/single/routing_strategy.py:100-150."""

    def __init__(self, hidden_size, num_experts, top_k=2, temperature=1.0):
        super().__init__()
        self.hidden_size, self.num_experts, self.top_k, self.temperature = hidden_size, num_experts, top_k, temperature
        self.load_balancing_router = LoadBalancingRouter(hidden_size, num_experts, top_k, temperature)
        self.importance_router = ImportanceAwareRouter(hidden_size, num_experts, top_k, temperature)
        self.router_selector = nn.Sequential(nn.Linear(hidden_size, hidden_size // 2), nn.ReLU(),
                                             nn.Linear(hidden_size // 2, 2), nn.Softmax(dim=-1))
        self.last_gate = None

    def forward(self, x, expert_mask=None):
        if x.dim() == 2:
            x = x.unsqueeze(-1).expand(-1, -1, self.hidden_size)
        elif x.dim() == 1:
            x = x.unsqueeze(0).unsqueeze(-1).expand(-1, -1, self.hidden_size)
        b, s, _ = x.shape
        sel = self.router_selector(x.mean(dim=1))
        lb_w, _, _, lb_loss = self.load_balancing_router(x, expert_mask)
        imp_w, _, _, importance = self.importance_router(x, expert_mask)
        routing_weights = sel[:, 0:1, None] * lb_w + sel[:, 1:2, None] * imp_w
        # top-k of the mixture on the kernel: logits = log(weights), softmax gives the weights back
        g = ops.gate_fused(logits=torch.log(routing_weights.reshape(-1, self.num_experts).float()).contiguous(),
                           top_k=self.top_k, want_probs=False)
        self.last_gate = g
        return (routing_weights, g.topk_idx.view(b, s, self.top_k).long(), g.topk_w.view(b, s, self.top_k), lb_loss,
                importance)
