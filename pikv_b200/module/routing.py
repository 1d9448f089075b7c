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


class AdaptiveRouter(BaseRouter):
    """core/single/module/pikv_routing.py:296-404: a sigmoid importance score per token, a predicted top-k
    for the whole batch, and combine weights doubled for tokens above the threshold."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 dropout: float = 0.0, importance_threshold: float = 0.5, adaptive_top_k: bool = True):
        super().__init__(hidden_size, num_experts, top_k, capacity_factor, dropout)
        self.importance_threshold = importance_threshold
        self.adaptive_top_k = adaptive_top_k
        self.importance_predictor = nn.Sequential(nn.Linear(hidden_size, hidden_size // 2), nn.ReLU(), nn.Dropout(dropout),
                                                  nn.Linear(hidden_size // 2, 1), nn.Sigmoid())
        if adaptive_top_k:
            self.top_k_predictor = nn.Sequential(nn.Linear(hidden_size + 1, hidden_size // 4), nn.ReLU(),
                                                 nn.Linear(hidden_size // 4, top_k), nn.Softmax(dim=-1))
        self.register_buffer("importance_history", torch.zeros(1000))
        self.register_buffer("importance_idx", torch.tensor(0))
        self._host_imp_idx: Optional[int] = None

    def _compute_importance(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.importance_predictor(hidden_states).squeeze(-1)

    def _adapt_top_k(self, hidden_states: torch.Tensor, importance: torch.Tensor) -> int:
        """:345-363.  One host read per call: the reference picks k with argmax(...).item()."""
        if not self.adaptive_top_k or not hasattr(self, "top_k_predictor"):
            return self.top_k
        feats = torch.cat([hidden_states.mean(dim=[0, 1]), importance.mean().unsqueeze(0)])
        return min(int(torch.argmax(self.top_k_predictor(feats)).item()) + 1, self.top_k)

    def _record_importance(self, importance: torch.Tensor) -> None:
        # :395-401 writes the values one by one into a ring of 1000; the last write to a position wins
        flat = importance.detach().flatten()
        n = flat.numel()
        if self._host_imp_idx is None:
            self._host_imp_idx = int(self.importance_idx.item())
        start = self._host_imp_idx
        if n > 1000:
            flat, start, n_w = flat[n - 1000:], start + n - 1000, 1000
        else:
            n_w = n
        pos = (start + torch.arange(n_w, device=flat.device)) % 1000
        self.importance_history[pos] = flat
        self.importance_idx += n
        self._host_imp_idx += n

    def forward(self, hidden_states: torch.Tensor, expert_mask: Optional[torch.Tensor] = None):
        b, s, _ = hidden_states.shape
        importance = self._compute_importance(hidden_states)
        k = self._adapt_top_k(hidden_states, importance)
        g, dispatch, combine = self._route(hidden_states, expert_mask, top_k=k)
        aux_loss = self._aux(g, b * s)
        with torch.no_grad():
            self.total_tokens += b * s
            cnt = g.counts.float()
            self.expert_usage_count += cnt
            self.routing_decisions += cnt
        weight = (importance > self.importance_threshold).float()
        combine = combine * (1.0 + weight[:, :, None, None])
        with torch.no_grad():
            self._record_importance(importance)
        return dispatch, combine, g.probs.view(b, s, self.num_experts), aux_loss, importance


class PiKVRouter(AdaptiveRouter):
    """core/single/module/pikv_routing.py:406-537: the router logits get a per-batch tanh adjustment computed
    from the mean hidden state and the experts' cache hit rates before the fused gate tail."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 dropout: float = 0.0, importance_threshold: float = 0.5, cache_aware: bool = True,
                 cache_update_interval: int = 100):
        super().__init__(hidden_size, num_experts, top_k, capacity_factor, dropout, importance_threshold, True)
        self.cache_aware = cache_aware
        self.cache_update_interval = cache_update_interval
        self.register_buffer("cache_usage_history", torch.zeros(num_experts, 100))
        self.register_buffer("cache_hit_rates", torch.zeros(num_experts))
        self.register_buffer("cache_update_counter", torch.tensor(0))
        if cache_aware:
            self.cache_router_adjustment = nn.Sequential(nn.Linear(hidden_size + num_experts, hidden_size), nn.ReLU(),
                                                         nn.Linear(hidden_size, num_experts), nn.Tanh())

    def update_cache_usage(self, expert_idx: int, cache_hit_rate: float):
        """:441-451."""
        if 0 <= expert_idx < self.num_experts:
            self.cache_hit_rates[expert_idx] = cache_hit_rate
            self.cache_usage_history[expert_idx, int(self.cache_update_counter.item()) % 100] = cache_hit_rate
        self.cache_update_counter += 1

    def _compute_cache_aware_adjustment(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        if not self.cache_aware or not hasattr(self, "cache_router_adjustment"):
            return torch.zeros_like(router_logits)
        b, s, _ = hidden_states.shape
        rates = self.cache_hit_rates.unsqueeze(0).expand(b, -1)
        adj = self.cache_router_adjustment(torch.cat([hidden_states.mean(dim=1), rates], dim=-1))
        return adj.unsqueeze(1).expand(-1, s, -1)

    def forward(self, hidden_states: torch.Tensor, kv_cache_states: Optional[torch.Tensor] = None,
                expert_mask: Optional[torch.Tensor] = None):
        b, s, _ = hidden_states.shape
        logits = self.router(hidden_states)
        if self.cache_aware:
            logits = logits + self._compute_cache_aware_adjustment(hidden_states, logits)
        importance = self._compute_importance(hidden_states)
        k = self._adapt_top_k(hidden_states, importance)
        # mask, softmax, top-k, renormalisation (+1e-8), running-count slots and counts: one fused call
        g, dispatch, combine = self._route(hidden_states, expert_mask, logits=logits, top_k=k)
        aux_loss = self._aux(g, b * s)
        with torch.no_grad():
            self.total_tokens += b * s
            self.expert_usage_count += g.counts.float()
        return dispatch, combine, g.probs.view(b, s, self.num_experts), aux_loss, importance
