"""H2O scheduler with the surface of core/single/module/pikv_scheduling.py:96-180: scores decay by
`attention_decay` before every accumulate, and nothing is evicted while the cache fits."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..scheduling import BaseScheduler


class H2OScheduler(BaseScheduler):
    def __init__(self, cache_size: int, hidden_size: int, heavy_ratio: float = 0.1, recent_ratio: float = 0.1,
                 attention_decay: float = 0.95):
        super().__init__(cache_size, hidden_size)
        self.heavy_ratio, self.recent_ratio, self.attention_decay = heavy_ratio, recent_ratio, attention_decay
        self.register_buffer("attention_accumulator", torch.zeros(cache_size))
        self.register_buffer("access_timestamps", torch.zeros(cache_size))
        self.register_buffer("current_time", torch.tensor(0))
        self._host_time: Optional[int] = None
        self.last_keep_idx = None
        self.last_kept_count = None

    def update_attention_scores(self, indices: torch.Tensor, attention_weights: torch.Tensor):
        if self._host_time is None:
            self._host_time = int(self.current_time.item())
        ops.h2o_accumulate(self.attention_accumulator, self.access_timestamps, indices.to(torch.int32),
                           attention_weights.to(torch.float32), float(self._host_time), decay=self.attention_decay)
        self._host_time += 1
        self.current_time += 1

    def select_eviction_candidates(self, keys: torch.Tensor, values: torch.Tensor,
                                   metadata: Dict[str, torch.Tensor]) -> torch.Tensor:
        cache_len = keys.size(0)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        # only reachable when the caller hands in more rows than the scheduler tracks
        n = self.attention_accumulator.numel()
        num_heavy = max(1, int(cache_len * self.heavy_ratio))
        num_recent = max(1, int(cache_len * self.recent_ratio))
        mask, keep, cnt = ops.h2o_select(self.attention_accumulator[:cache_len].contiguous(),
                                         self.access_timestamps[:cache_len].contiguous(), min(num_heavy, n),
                                         min(num_recent, n))
        self.last_keep_idx, self.last_kept_count = keep[0], cnt
        out = torch.ones(cache_len, dtype=torch.bool, device=keys.device)
        out[: mask.shape[1]] = mask[0]
        return out
