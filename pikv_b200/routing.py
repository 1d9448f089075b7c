"""Routers with the constructor / forward surface of core/single/pikv_routing.py.

Same class names, keyword arguments, parameter and buffer names (state_dicts of
the reference load unchanged) and return tuples.  The gate net's hidden layer
stays a torch (cuBLAS) GEMM; everything after it - last-layer logits, mask,
softmax, top-k, renormalisation, per-expert counts and slot assignment - is one
call of the fused CUDA gate kernel.  The dense dispatch / combine tensors the
reference returns are produced by a scatter kernel from the compact result,
which stays available as `router.last_gate`.

Modules must live on a CUDA device; there is no CPU path.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, ops


def _aux_base(p_mean: torch.Tensor, num_experts: int) -> torch.Tensor:
    # core/single/pikv_routing.py:155-159
    return torch.sum(p_mean * torch.log(p_mean * num_experts + 1e-9))


class BaseRouter(nn.Module):
    """core/single/pikv_routing.py:7-161."""

    #: how dispatch positions are formed: 1 = the positions core/single produces, 0 = running count
    position_mode = 1
    mask_mode = _lib.MASK_SINGLE
    renorm_eps = 0.0

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 expert_backend: str = "fairscale"):
        super().__init__()
        self.hidden_size = hidden_size
        self.num_experts = num_experts
        self.top_k = min(top_k, num_experts)
        self.capacity_factor = capacity_factor
        self.expert_backend = expert_backend
        self.router = nn.Sequential(nn.Linear(hidden_size, hidden_size), nn.ReLU(), nn.Linear(hidden_size, num_experts))
        self.last_gate: Optional[ops.GateResult] = None

    def _compute_capacity(self, batch_size: int, seq_len: int) -> int:
        return int(batch_size * seq_len * self.capacity_factor * self.top_k / self.num_experts)

    # -- shared machinery -----------------------------------------------------------
    def _gate(self, act2d: Optional[torch.Tensor], last: Optional[nn.Linear], *, logits: Optional[torch.Tensor] = None,
              expert_mask=None, correction=None, capacity: int = 0, top_k: Optional[int] = None) -> ops.GateResult:
        k = self.top_k if top_k is None else top_k
        if logits is not None:
            g = ops.gate_fused(logits=logits, top_k=k, expert_mask=expert_mask, mask_mode=self.mask_mode,
                               correction=correction, renorm_eps=self.renorm_eps, capacity=capacity)
        else:
            g = ops.gate_fused(act2d, last.weight.detach().to(act2d.dtype), last.bias.detach() if last.bias is not None else None,
                               top_k=k, expert_mask=expert_mask, mask_mode=self.mask_mode, correction=correction,
                               renorm_eps=self.renorm_eps, capacity=capacity)
        self.last_gate = g
        return g

    def _dense(self, g: ops.GateResult, batch_size: int, seq_len: int, capacity: int):
        if self.expert_backend == "fairscale":
            d, c = ops.dispatch_scatter(g, self.num_experts, capacity, self.position_mode)
            return (d.view(batch_size, seq_len, self.num_experts, capacity),
                    c.view(batch_size, seq_len, self.num_experts, capacity))
        # the "basic" backend of the reference: capacity dimension of 1, every choice written to position 0
        T, k = g.topk_idx.shape
        d = torch.zeros(T, self.num_experts, dtype=torch.float32, device=g.topk_idx.device)
        c = torch.zeros_like(d)
        idx = g.topk_idx.long()
        d.scatter_(1, idx, 1.0)
        c.scatter_(1, idx, g.topk_w)
        return (d.view(batch_size, seq_len, self.num_experts, 1), c.view(batch_size, seq_len, self.num_experts, 1))

    def _hidden(self, mlp: nn.Sequential, x2d: torch.Tensor) -> torch.Tensor:
        return F.relu(mlp[0](x2d))

    def _gate_net(self, mlp: nn.Sequential, x2d: torch.Tensor, **kw) -> ops.GateResult:
        """Gate net + tail.  bf16 inputs: one tensor-core kernel for both layers and the tail (the hidden
        activations stay on chip).  fp32 inputs (the reference's dtype, 1e-5 parity): the first layer is a torch
        fp32 GEMM and the kernel takes over from the hidden activations."""
        if x2d.dtype == torch.bfloat16 and self.num_experts <= 32 and x2d.shape[1] % 8 == 0 and mlp[0].out_features % 8 == 0:
            k = kw.pop("top_k", None) or self.top_k
            first, last = mlp[0], mlp[2]
            g = ops.gate_mlp_fused(x2d, first.weight.detach().to(torch.bfloat16),
                                   None if first.bias is None else first.bias.detach(),
                                   last.weight.detach().to(torch.bfloat16), None if last.bias is None else last.bias.detach(),
                                   top_k=k, mask_mode=self.mask_mode, renorm_eps=self.renorm_eps, **kw)
            self.last_gate = g
            return g
        return self._gate(self._hidden(mlp, x2d), mlp[2], **kw)

    def forward(self, hidden_states: torch.Tensor, expert_mask: Optional[torch.Tensor] = None):
        batch_size, seq_len, hidden_size = hidden_states.shape
        x2d = hidden_states.reshape(-1, hidden_size)
        capacity = self._compute_capacity(batch_size, seq_len)
        g = self._gate_net(self.router, x2d, expert_mask=expert_mask, capacity=capacity)
        dispatch, combine = self._dense(g, batch_size, seq_len, max(capacity, 1))
        p_mean = g.prob_sum / float(batch_size * seq_len)
        aux_loss = _aux_base(p_mean, self.num_experts)
        return dispatch, combine, g.probs.view(batch_size, seq_len, self.num_experts), aux_loss


class TopKBalancedRouter(BaseRouter):
    """core/single/pikv_routing.py:163-222."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 expert_backend: str = "fairscale", balance_coefficient: float = 0.01, balance_mode: str = "entropy"):
        super().__init__(hidden_size, num_experts, top_k, capacity_factor, expert_backend)
        self.balance_coefficient = balance_coefficient
        self.balance_mode = balance_mode

    def forward(self, hidden_states: torch.Tensor, expert_mask: Optional[torch.Tensor] = None):
        dispatch, combine, probs, aux_loss = super().forward(hidden_states, expert_mask)
        p = self.last_gate.prob_sum / float(hidden_states.shape[0] * hidden_states.shape[1])
        if self.balance_mode == "entropy":
            term = -torch.sum(p * torch.log(p + 1e-9)) / math.log(self.num_experts)
            balance = -self.balance_coefficient * term
        elif self.balance_mode == "cv":
            balance = self.balance_coefficient * (p.std() / (p.mean() + 1e-9))
        else:
            uniform = torch.ones_like(p) / self.num_experts
            balance = self.balance_coefficient * torch.sum((p - uniform) ** 2)
        return dispatch, combine, probs, aux_loss + balance


class AdaptiveRouter(BaseRouter):
    """core/single/pikv_routing.py:224-377."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 expert_backend: str = "fairscale", imp_threshold: float = 0.5):
        super().__init__(hidden_size, num_experts, top_k, capacity_factor, expert_backend)
        self.importance_predictor = nn.Sequential(nn.Linear(hidden_size, hidden_size // 2), nn.ReLU(),
                                                  nn.Linear(hidden_size // 2, 1), nn.Sigmoid())
        self.imp_threshold = imp_threshold
        self.router_important = nn.Sequential(nn.Linear(hidden_size, hidden_size), nn.ReLU(),
                                              nn.Linear(hidden_size, num_experts))
        self.router_unimportant = nn.Sequential(nn.Linear(hidden_size, hidden_size), nn.ReLU(),
                                                nn.Linear(hidden_size, num_experts))

    def _blended_logits(self, hidden_states: torch.Tensor, importance: torch.Tensor):
        imp_mask = (importance > self.imp_threshold).float()
        logits = imp_mask * self.router_important(hidden_states) + (1 - imp_mask) * self.router_unimportant(hidden_states)
        return logits, imp_mask

    def forward(self, hidden_states: torch.Tensor, expert_mask: Optional[torch.Tensor] = None):
        batch_size, seq_len, hidden_size = hidden_states.shape
        importance = self.importance_predictor(hidden_states)
        logits, imp_mask = self._blended_logits(hidden_states, importance)
        capacity = self._compute_capacity(batch_size, seq_len)
        g = self._gate(None, None, logits=logits.reshape(-1, self.num_experts).float(), expert_mask=expert_mask,
                       capacity=capacity)
        dispatch, combine = self._dense(g, batch_size, seq_len, max(capacity, 1))
        probs = g.probs.view(batch_size, seq_len, self.num_experts)
        p_mean = g.prob_sum / float(batch_size * seq_len)
        entropy_loss = _aux_base(p_mean, self.num_experts)
        imp_sum = (probs * imp_mask).sum(dim=[0, 1]) + 1e-9             # :365-372
        imp_per = imp_sum / imp_sum.sum()
        imp_entropy = -torch.sum(imp_per * torch.log(imp_per + 1e-9)) / math.log(self.num_experts)
        return dispatch, combine, probs, entropy_loss + (-0.1 * imp_entropy), importance


class PiKVRouter(AdaptiveRouter):
    """core/single/pikv_routing.py:379-549."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.5,
                 expert_backend: str = "fairscale", imp_threshold: float = 0.5, cache_update_interval: int = 100):
        super().__init__(hidden_size, num_experts, top_k, capacity_factor, expert_backend, imp_threshold)
        self.register_buffer("cache_usage_history", torch.zeros(num_experts))
        self.kv_importance_model = nn.Sequential(nn.Linear(hidden_size, hidden_size // 2), nn.ReLU(),
                                                 nn.Linear(hidden_size // 2, 1), nn.Sigmoid())
        self.cache_correction_factor = nn.Parameter(torch.ones(num_experts))
        self.register_buffer("update_counter", torch.tensor(0))
        self.cache_update_interval = cache_update_interval
        self._host_counter: Optional[int] = None   # host mirror of update_counter: no device sync per call

    def update_cache_usage(self, usage_vector: torch.Tensor):
        self.cache_usage_history = 0.9 * self.cache_usage_history + 0.1 * usage_vector
        if self._host_counter is None:
            self._host_counter = int(self.update_counter.item())
        self.update_counter += 1
        self._host_counter += 1
        if self._host_counter % self.cache_update_interval == 0:
            factor = 1.0 / (self.cache_usage_history + 0.5)
            self.cache_correction_factor.data = factor / factor.mean()

    def _load_from_state_dict(self, *args, **kwargs):
        self._host_counter = None
        return super()._load_from_state_dict(*args, **kwargs)

    def forward(self, hidden_states: torch.Tensor, kv_states: Optional[torch.Tensor] = None,
                expert_mask: Optional[torch.Tensor] = None):
        batch_size, seq_len, hidden_size = hidden_states.shape
        importance = self.importance_predictor(hidden_states)
        if kv_states is not None:
            importance = (importance + self.kv_importance_model(kv_states)) / 2
        logits, _ = self._blended_logits(hidden_states, importance)
        capacity = self._compute_capacity(batch_size, seq_len)
        g = self._gate(None, None, logits=logits.reshape(-1, self.num_experts).float(), expert_mask=expert_mask,
                       correction=self.cache_correction_factor.detach(), capacity=capacity)
        dispatch, combine = self._dense(g, batch_size, seq_len, max(capacity, 1))
        probs = g.probs.view(batch_size, seq_len, self.num_experts)
        usage_norm = g.prob_sum / g.prob_sum.sum()
        self.update_cache_usage(usage_norm)
        p_mean = g.prob_sum / float(batch_size * seq_len)
        aux_loss = _aux_base(p_mean, self.num_experts) + 0.05 * torch.sum(self.cache_usage_history * usage_norm)
        return dispatch, combine, probs, aux_loss, importance
