"""Routers with the surface of core/single/module/pikv_routing.py: running-count dispatch
positions, usage counters, E * sum(p_mean * usage_rate) auxiliary loss."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib, ops


class BaseRouter(nn.Module):
    """core/single/module/pikv_routing.py:19-201."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 dropout: float = 0.0):
        super().__init__()
        self.hidden_size = hidden_size
        self.num_experts = num_experts
        self.top_k = min(top_k, num_experts)
        self.capacity_factor = capacity_factor
        self.dropout = dropout
        self.router = nn.Sequential(nn.Linear(hidden_size, hidden_size), nn.ReLU(), nn.Dropout(dropout),
                                    nn.Linear(hidden_size, num_experts))
        self.register_buffer("total_tokens", torch.tensor(0.0))
        self.register_buffer("expert_usage_count", torch.zeros(num_experts))
        self.register_buffer("routing_decisions", torch.zeros(num_experts))
        for m in self.router:
            if isinstance(m, nn.Linear):
                nn.init.xavier_normal_(m.weight)
                nn.init.zeros_(m.bias)
        self.last_gate: Optional[ops.GateResult] = None

    def _compute_capacity(self, batch_size: int, seq_len: int) -> int:
        return int(batch_size * seq_len * self.capacity_factor * self.top_k / self.num_experts)

    def _route(self, hidden_states, expert_mask, logits=None, top_k=None):
        b, s, h = hidden_states.shape
        k = self.top_k if top_k is None else top_k
        cap = int(b * s * self.capacity_factor * k / self.num_experts)
        if logits is None:
            act = self.router[2](F.relu(self.router[0](hidden_states.reshape(-1, h))))
            last = self.router[3]
            g = ops.gate_fused(act, last.weight.detach().to(act.dtype), last.bias.detach(), top_k=k,
                               expert_mask=expert_mask, mask_mode=_lib.MASK_MODULE, renorm_eps=1e-8, capacity=cap)
        else:
            g = ops.gate_fused(logits=logits.reshape(-1, self.num_experts).float(), top_k=k, expert_mask=expert_mask,
                               mask_mode=_lib.MASK_MODULE, renorm_eps=1e-8, capacity=cap)
        self.last_gate = g
        d, c = ops.dispatch_scatter(g, self.num_experts, max(cap, 1), position_mode=0)
        shape = (b, s, self.num_experts, max(cap, 1))
        return g, d.view(shape), c.view(shape)

    def _aux(self, g: ops.GateResult, tokens: int) -> torch.Tensor:
        # :164-181: E * sum(p_mean * mean(one_hot(top-k)))
        usage = g.counts.float() / float(tokens * g.topk_idx.shape[1])
        return torch.sum(g.prob_sum / float(tokens) * usage) * self.num_experts

    def forward(self, hidden_states: torch.Tensor, expert_mask: Optional[torch.Tensor] = None):
        b, s, _ = hidden_states.shape
        g, dispatch, combine = self._route(hidden_states, expert_mask)
        aux_loss = self._aux(g, b * s)
        with torch.no_grad():
            self.total_tokens += b * s
            cnt = g.counts.float()
            self.expert_usage_count += cnt
            self.routing_decisions += cnt
        return dispatch, combine, g.probs.view(b, s, self.num_experts), aux_loss

    def get_routing_stats(self) -> Dict[str, torch.Tensor]:
        ratios = self.expert_usage_count / self.total_tokens if self.total_tokens > 0 else torch.zeros_like(self.expert_usage_count)
        return {"expert_usage_ratios": ratios, "expert_usage_count": self.expert_usage_count,
                "total_tokens": self.total_tokens, "routing_decisions": self.routing_decisions}

    def reset_stats(self):
        self.total_tokens.zero_()
        self.expert_usage_count.zero_()
        self.routing_decisions.zero_()


class TopKBalancedRouter(BaseRouter):
    """core/single/module/pikv_routing.py:203-294."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 dropout: float = 0.0, balance_coefficient: float = 0.01, balance_mode: str = "entropy"):
        super().__init__(hidden_size, num_experts, top_k, capacity_factor, dropout)
        self.balance_coefficient = balance_coefficient
        self.balance_mode = balance_mode
        self.register_buffer("balance_loss_history", torch.zeros(100))
        self.register_buffer("balance_loss_idx", torch.tensor(0))
        self._host_idx: Optional[int] = None

    def _advanced(self, p: torch.Tensor) -> torch.Tensor:
        if self.balance_mode == "entropy":
            return 1.0 - (-torch.sum(p * torch.log(p + 1e-8)) / math.log(self.num_experts))
        if self.balance_mode == "variance":
            return torch.var(p - 1.0 / self.num_experts)
        if self.balance_mode == "gini":
            sp, _ = torch.sort(p)
            index = torch.arange(1, self.num_experts + 1, dtype=torch.float, device=p.device)
            return (2 * torch.sum(index * sp) / (self.num_experts * torch.sum(sp))) - 1
        raise ValueError(f"balance_mode {self.balance_mode!r}")

    def forward(self, hidden_states: torch.Tensor, expert_mask: Optional[torch.Tensor] = None):
        dispatch, combine, probs, base = super().forward(hidden_states, expert_mask)
        tokens = hidden_states.shape[0] * hidden_states.shape[1]
        adv = self._advanced(self.last_gate.prob_sum / float(tokens))
        with torch.no_grad():
            if self._host_idx is None:
                self._host_idx = int(self.balance_loss_idx.item())
            self.balance_loss_history[self._host_idx % 100] = adv
            self.balance_loss_idx += 1
            self._host_idx += 1
        return dispatch, combine, probs, base + self.balance_coefficient * adv
