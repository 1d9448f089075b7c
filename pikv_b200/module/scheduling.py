"""Schedulers with the surface of core/single/module/pikv_scheduling.py: the H2O variant (:96-180: scores
decay by `attention_decay` before every accumulate, nothing is evicted while the cache fits), AdaKV
(:624-672) and DuoAttention (:674-710).  Every "keep the m best" choice runs on the segmented select
kernel (ties go to the lowest index)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

import torch.nn as nn

from .. import ops
from ..scheduling import BaseScheduler as _SingleBaseScheduler


class BaseScheduler(_SingleBaseScheduler):
    """core/single/module/pikv_scheduling.py:33-93: the single-file base plus an operation counter."""

    def __init__(self, cache_size: int, hidden_size: int):
        super().__init__(cache_size, hidden_size)
        self.register_buffer("total_operations", torch.tensor(0))

    def get_eviction_rate(self):
        return self.eviction_count.float() / self.total_operations.float() if self.total_operations > 0 else 0.0

    def reset_stats(self):
        super().reset_stats()
        self.total_operations.zero_()

    def update_stats(self, hit: bool = False, miss: bool = False, eviction: bool = False):
        if hit:
            self.hit_count += 1
        if miss:
            self.miss_count += 1
        if eviction:
            self.eviction_count += 1
        self.total_operations += 1

    def get_scheduler_stats(self) -> Dict[str, float]:
        hr, er = self.get_hit_rate(), self.get_eviction_rate()
        return {"hit_rate": float(hr), "eviction_rate": float(er), "total_hits": self.hit_count.item(),
                "total_misses": self.miss_count.item(), "total_evictions": self.eviction_count.item(),
                "total_operations": self.total_operations.item()}


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


class AdaKVScheduler(BaseScheduler):
    """core/single/module/pikv_scheduling.py:624-672: keep the int(n * (1 - compression_ratio)) rows with the
    highest linear importance score.  The reference picks a safeguarded head of that set first and the rest
    second; both picks are top-k by the same score, so the union is one top-k, which is what the select
    kernel computes (in one pass, ties to the lowest index).  Only the first cache_size rows carry scores:
    rows past them are always evicted, as in the reference."""

    def __init__(self, cache_size: int, hidden_size: int, compression_ratio: float = 0.5, safeguard_ratio: float = 0.2):
        super().__init__(cache_size, hidden_size)
        self.compression_ratio, self.safeguard_ratio = compression_ratio, safeguard_ratio
        self.register_buffer("importance_scores", torch.zeros(cache_size))
        self.linear_proj = nn.Linear(hidden_size, 1)

    def update_importance(self, indices: torch.Tensor, keys: torch.Tensor):
        self.importance_scores[indices] = self.linear_proj(keys).squeeze(-1)

    def select_eviction_candidates(self, keys, values, metadata) -> torch.Tensor:
        cache_len = keys.size(0)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        scores = self.importance_scores[:cache_len].detach().contiguous()
        num_keep = int(cache_len * (1 - self.compression_ratio))
        if num_keep > scores.numel():
            raise RuntimeError(f"selected index k out of range: keep {num_keep} of {scores.numel()} scored rows")
        mask = torch.ones(cache_len, dtype=torch.bool, device=keys.device)
        if num_keep > 0:
            kept, _, _ = ops.h2o_select(scores[None], scores[None], num_keep, 0, want_idx=False)
            mask[: scores.numel()] = kept[0]
        self.update_stats(eviction=True)
        return mask

    def get_scheduler_stats(self) -> Dict[str, float]:
        stats = super().get_scheduler_stats()
        stats.update({"compression_ratio": self.compression_ratio, "safeguard_ratio": self.safeguard_ratio})
        return stats


class DuoAttentionScheduler(BaseScheduler):
    """core/single/module/pikv_scheduling.py:674-710: keep the first sink_size and the last recent_size rows.
    Runs on the select kernel with the position as the key: the sink rows are the sink_size largest of
    -position, the recent rows the recent_size largest of +position."""

    def __init__(self, cache_size: int, hidden_size: int, sink_size: int = 64, recent_size: int = 512):
        super().__init__(cache_size, hidden_size)
        self.sink_size, self.recent_size = sink_size, recent_size

    def select_eviction_candidates(self, keys, values, metadata) -> torch.Tensor:
        cache_len = keys.size(0)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        pos = torch.arange(cache_len, dtype=torch.float32, device=keys.device)[None]
        # python slicing: [:0] keeps nothing, [-0:] keeps everything
        recent = cache_len if self.recent_size == 0 else min(self.recent_size, cache_len)
        mask, _, _ = ops.h2o_select((-pos).contiguous(), pos, min(self.sink_size, cache_len), recent, want_idx=False)
        self.update_stats(eviction=bool(mask.any().item()))
        return mask[0]

    def get_scheduler_stats(self) -> Dict[str, float]:
        stats = super().get_scheduler_stats()
        stats.update({"sink_size": self.sink_size, "recent_size": self.recent_size})
        return stats
