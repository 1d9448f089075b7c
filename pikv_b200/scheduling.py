"""H2O scheduling with the surface of core/single/cache_scheduling.py.

H2OScheduler.select_eviction_candidates runs the segmented top-k CUDA kernel
(ties go to the lowest index, which torch.topk does not promise);
update_attention_scores runs the accumulate kernel.  CacheSchedulingManager
keeps the reference's evict-then-append behaviour, including the truncation of
new rows beyond capacity, and - unlike the reference - moves the scheduler's
scores and timestamps together with the rows it keeps.
"""
from __future__ import annotations

from enum import Enum
from typing import Dict, Optional

import torch
import torch.nn as nn

from . import ops


class SchedulingPolicy(Enum):
    """core/single/cache_scheduling.py:9-17.  Only NONE and H2O are served by this package."""
    NONE = "none"
    H2O = "h2o"
    STREAMING_LLM = "streaming_llm"
    QUEST = "quest"
    FLEXGEN = "flexgen"
    LRU = "lru"
    LRU_PLUS = "lru_plus"


class BaseScheduler(nn.Module):
    """core/single/cache_scheduling.py:19-51."""

    def __init__(self, cache_size: int, hidden_size: int):
        super().__init__()
        self.cache_size = cache_size
        self.hidden_size = hidden_size
        self.register_buffer("hit_count", torch.tensor(0))
        self.register_buffer("miss_count", torch.tensor(0))
        self.register_buffer("eviction_count", torch.tensor(0))

    def get_hit_rate(self) -> float:
        total = self.hit_count + self.miss_count
        return self.hit_count.float() / total.float() if total > 0 else 0.0

    def reset_stats(self):
        self.hit_count.zero_()
        self.miss_count.zero_()
        self.eviction_count.zero_()


class H2OScheduler(BaseScheduler):
    """core/single/cache_scheduling.py:53-99."""

    def __init__(self, cache_size: int, hidden_size: int, heavy_ratio: float = 0.1, recent_ratio: float = 0.1):
        super().__init__(cache_size, hidden_size)
        self.heavy_ratio = heavy_ratio
        self.recent_ratio = recent_ratio
        self.register_buffer("attention_accumulator", torch.zeros(cache_size))
        self.register_buffer("access_timestamps", torch.zeros(cache_size))
        self.register_buffer("current_time", torch.tensor(0))
        self._host_time: Optional[int] = None
        self.last_keep_idx = None
        self.last_kept_count = None

    def _load_from_state_dict(self, *args, **kwargs):
        self._host_time = None
        return super()._load_from_state_dict(*args, **kwargs)

    def update_attention_scores(self, indices: torch.Tensor, attention_weights: torch.Tensor):
        """acc[indices] += w ; ts[indices] = t ; t += 1 (:69-73).  Indices must be distinct."""
        if self._host_time is None:
            self._host_time = int(self.current_time.item())
        ops.h2o_accumulate(self.attention_accumulator, self.access_timestamps, indices.to(torch.int32),
                           attention_weights.to(torch.float32), float(self._host_time))
        self._host_time += 1
        self.current_time += 1

    def select_eviction_candidates(self, keys: torch.Tensor, values: torch.Tensor,
                                   metadata: Dict[str, torch.Tensor]) -> torch.Tensor:
        cache_len = keys.size(0)
        num_heavy = max(1, int(cache_len * self.heavy_ratio))
        num_recent = max(1, int(cache_len * self.recent_ratio))
        mask, keep, cnt = ops.h2o_select(self.attention_accumulator[:cache_len].contiguous(),
                                         self.access_timestamps[:cache_len].contiguous(), num_heavy, num_recent)
        self.last_keep_idx, self.last_kept_count = keep[0], cnt
        return mask[0]


class CacheSchedulingManager(nn.Module):
    """core/single/cache_scheduling.py:351-468."""

    def __init__(self, cache_size: int, hidden_size: int, policy: SchedulingPolicy = SchedulingPolicy.NONE):
        super().__init__()
        self.cache_size = cache_size
        self.hidden_size = hidden_size
        self.policy = policy
        self.scheduler = self._create_scheduler(policy)
        self.register_buffer("cache_keys", torch.zeros(cache_size, hidden_size))
        self.register_buffer("cache_values", torch.zeros(cache_size, hidden_size))
        self.register_buffer("cache_valid", torch.zeros(cache_size, dtype=torch.bool))
        self.register_buffer("cache_size_current", torch.tensor(0))
        self._host_size: Optional[int] = None

    def _create_scheduler(self, policy: SchedulingPolicy):
        if policy == SchedulingPolicy.NONE:
            return None
        if policy == SchedulingPolicy.H2O:
            return H2OScheduler(self.cache_size, self.hidden_size)
        raise ValueError(f"scheduling policy {policy} is not served by pikv_b200 (NONE and H2O are)")

    def _load_from_state_dict(self, *args, **kwargs):
        self._host_size = None
        return super()._load_from_state_dict(*args, **kwargs)

    def _size(self) -> int:
        if self._host_size is None:
            self._host_size = int(self.cache_size_current.item())
        return self._host_size

    def update_cache(self, keys: torch.Tensor, values: torch.Tensor, metadata: Optional[Dict[str, torch.Tensor]] = None):
        if self.scheduler is None:
            return
        hidden = keys.shape[-1]
        kf, vf = keys.reshape(-1, hidden), values.reshape(-1, hidden)
        new_items = kf.size(0)
        cur = self._size()
        if cur + new_items > self.cache_size:
            sch = self.scheduler
            evict = sch.select_eviction_candidates(self.cache_keys[:cur], self.cache_values[:cur], metadata or {})
            kept = int(sch.last_kept_count.item())          # one host read per eviction, as the reference's len()
            keep = sch.last_keep_idx[:kept].long()
            self.cache_keys[:kept] = self.cache_keys[keep]
            self.cache_values[:kept] = self.cache_values[keep]
            # the scores travel with their rows (the reference leaves them behind, :422-423)
            sch.attention_accumulator[:kept] = sch.attention_accumulator[keep]
            sch.access_timestamps[:kept] = sch.access_timestamps[keep]
            sch.attention_accumulator[kept:cur] = 0
            sch.access_timestamps[kept:cur] = 0
            sch.eviction_count += cur - kept
            cur = kept
        end = min(cur + new_items, self.cache_size)
        self.cache_keys[cur:end] = kf[: end - cur]
        self.cache_values[cur:end] = vf[: end - cur]
        self.cache_size_current.fill_(end)
        self._host_size = end

    def get_cache_stats(self) -> Dict[str, float]:
        stats = {"cache_size": self._size(), "cache_utilization": self._size() / self.cache_size,
                 "policy": self.policy.value}
        if self.scheduler is not None:
            stats.update({"hit_rate": self.scheduler.get_hit_rate(), "eviction_count": self.scheduler.eviction_count.item()})
        return stats

    def reset_cache(self):
        self.cache_keys.zero_()
        self.cache_values.zero_()
        self.cache_valid.zero_()
        self.cache_size_current.zero_()
        self._host_size = 0
        if self.scheduler is not None:
            self.scheduler.reset_stats()

    def change_policy(self, new_policy: SchedulingPolicy):
        self.policy = new_policy
        self.scheduler = self._create_scheduler(new_policy)
        if self.scheduler is not None:
            self.scheduler.to(self.cache_keys.device)
        self.reset_cache()
