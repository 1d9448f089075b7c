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
    """core/single/cache_scheduling.py:9-17."""
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


def _evict_lowest(scores: torch.Tensor, num_to_evict: int, cache_len: int) -> torch.Tensor:
    """bool [cache_len]: True at the num_to_evict lowest scores (ties: lowest index first).  The segmented select
    kernel keeps the m largest keys, so it runs on the negated scores and its kept set is the evicted one."""
    n = scores.numel()
    mask = torch.zeros(cache_len, dtype=torch.bool, device=scores.device)
    if num_to_evict <= 0 or n == 0:
        return mask
    if num_to_evict > n:
        raise ValueError(f"cannot evict {num_to_evict} of {n} scored entries")
    neg = (-scores.float()).contiguous()[None]
    not_kept, _, _ = ops.h2o_select(neg, neg, num_to_evict, 0, want_idx=False)
    mask[:n] = ~not_kept[0]
    return mask


class StreamingLLMScheduler(BaseScheduler):
    """core/single/cache_scheduling.py:101-133: keep the first start_size entries and the last recent_size."""

    def __init__(self, cache_size: int, hidden_size: int, start_size: int = 4, recent_size: Optional[int] = None):
        super().__init__(cache_size, hidden_size)
        self.start_size = start_size
        self.recent_size = recent_size if recent_size is not None else (cache_size - start_size)
        self.register_buffer("position_counter", torch.tensor(0))

    def select_eviction_candidates(self, keys, values, metadata) -> torch.Tensor:
        cache_len = keys.size(0)
        pos = torch.arange(cache_len, device=keys.device)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        recent_start = max(self.start_size, cache_len - self.recent_size)
        return (pos >= self.start_size) & (pos < recent_start)


class LRUScheduler(BaseScheduler):
    """core/single/cache_scheduling.py:254-286: evict the entries with the oldest access times."""

    def __init__(self, cache_size: int, hidden_size: int):
        super().__init__(cache_size, hidden_size)
        self.register_buffer("access_times", torch.zeros(cache_size))
        self.register_buffer("global_time", torch.tensor(0))

    def update_access_time(self, indices: torch.Tensor):
        self.access_times[indices] = self.global_time.to(self.access_times.dtype)
        self.global_time += 1

    def select_eviction_candidates(self, keys, values, metadata) -> torch.Tensor:
        cache_len = keys.size(0)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        return _evict_lowest(self.access_times[:cache_len], cache_len - self.cache_size, cache_len)


class LRUPlusScheduler(BaseScheduler):
    """core/single/cache_scheduling.py:288-349: priority = recency, frequency and importance mixed; the lowest go."""

    def __init__(self, cache_size: int, hidden_size: int, frequency_weight: float = 0.3, importance_weight: float = 0.4):
        super().__init__(cache_size, hidden_size)
        self.frequency_weight = frequency_weight
        self.importance_weight = importance_weight
        self.recency_weight = 1.0 - frequency_weight - importance_weight
        self.register_buffer("access_times", torch.zeros(cache_size))
        self.register_buffer("access_frequency", torch.zeros(cache_size))
        self.register_buffer("importance_scores", torch.zeros(cache_size))
        self.register_buffer("global_time", torch.tensor(0))

    def update_access_info(self, indices: torch.Tensor, importance: torch.Tensor):
        self.access_times[indices] = self.global_time.to(self.access_times.dtype)
        self.access_frequency[indices] += 1
        self.importance_scores[indices] = importance
        self.global_time += 1

    def compute_priority_scores(self, cache_len: int) -> torch.Tensor:
        t, f = self.access_times[:cache_len], self.access_frequency[:cache_len]
        recency = t / (t.max() + 1e-8)
        frequency = f / (f.max() + 1e-8)
        return (self.recency_weight * recency + self.frequency_weight * frequency +
                self.importance_weight * self.importance_scores[:cache_len])

    def select_eviction_candidates(self, keys, values, metadata) -> torch.Tensor:
        cache_len = keys.size(0)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        return _evict_lowest(self.compute_priority_scores(cache_len), cache_len - self.cache_size, cache_len)


class QUESTScheduler(BaseScheduler):
    """core/single/cache_scheduling.py:135-203: utility = quality x frequency x decay^age; everything under the
    threshold goes, or the lowest num_to_evict when those are too few."""

    def __init__(self, cache_size: int, hidden_size: int, quality_threshold: float = 0.1, decay_factor: float = 0.95):
        super().__init__(cache_size, hidden_size)
        self.quality_threshold = quality_threshold
        self.decay_factor = decay_factor
        self.register_buffer("quality_scores", torch.zeros(cache_size))
        self.register_buffer("usage_frequency", torch.zeros(cache_size))
        self.register_buffer("last_access_time", torch.zeros(cache_size))
        self.register_buffer("global_time", torch.tensor(0))

    def update_quality_scores(self, indices: torch.Tensor, reconstruction_errors: torch.Tensor):
        self.quality_scores[indices] = 1.0 / (1.0 + reconstruction_errors)
        self.usage_frequency[indices] += 1
        self.last_access_time[indices] = self.global_time.to(self.last_access_time.dtype)
        self.global_time += 1

    def compute_utility_scores(self, cache_len: int) -> torch.Tensor:
        decay = torch.pow(self.decay_factor, self.global_time - self.last_access_time[:cache_len])
        return self.quality_scores[:cache_len] * self.usage_frequency[:cache_len] * decay

    def select_eviction_candidates(self, keys, values, metadata) -> torch.Tensor:
        cache_len = keys.size(0)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        utility = self.compute_utility_scores(cache_len)
        below = utility < self.quality_threshold            # as long as the scored entries, like the reference's
        num_to_evict = cache_len - self.cache_size
        if int(below.sum().item()) < num_to_evict:          # one host read, as the reference's comparison
            return _evict_lowest(utility, num_to_evict, cache_len)
        return below


class FlexGenScheduler(BaseScheduler):
    """core/single/cache_scheduling.py:205-252: benefit = access frequency / access cost; the lowest go."""

    def __init__(self, cache_size: int, hidden_size: int, gpu_ratio: float = 0.3, cpu_ratio: float = 0.5):
        super().__init__(cache_size, hidden_size)
        self.gpu_ratio, self.cpu_ratio = gpu_ratio, cpu_ratio
        self.gpu_cache_size = int(cache_size * gpu_ratio)
        self.cpu_cache_size = int(cache_size * cpu_ratio)
        self.disk_cache_size = cache_size - self.gpu_cache_size - self.cpu_cache_size
        self.register_buffer("access_frequency", torch.zeros(cache_size))
        self.register_buffer("access_cost", torch.ones(cache_size))
        self.register_buffer("cache_level", torch.zeros(cache_size, dtype=torch.long))

    def update_access_patterns(self, indices: torch.Tensor, access_costs: torch.Tensor):
        self.access_frequency[indices] += 1
        self.access_cost[indices] = access_costs

    def select_eviction_candidates(self, keys, values, metadata) -> torch.Tensor:
        cache_len = keys.size(0)
        if cache_len <= self.cache_size:
            return torch.zeros(cache_len, dtype=torch.bool, device=keys.device)
        benefit = self.access_frequency[:cache_len] / self.access_cost[:cache_len]
        return _evict_lowest(benefit, cache_len - self.cache_size, cache_len)


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
        classes = {SchedulingPolicy.H2O: H2OScheduler, SchedulingPolicy.STREAMING_LLM: StreamingLLMScheduler,
                   SchedulingPolicy.QUEST: QUESTScheduler, SchedulingPolicy.FLEXGEN: FlexGenScheduler,
                   SchedulingPolicy.LRU: LRUScheduler, SchedulingPolicy.LRU_PLUS: LRUPlusScheduler}
        if policy not in classes:
            raise ValueError(f"Unknown scheduling policy: {policy}")
        return classes[policy](self.cache_size, self.hidden_size)

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
            if isinstance(sch, H2OScheduler):
                kept = int(sch.last_kept_count.item())      # one host read per eviction, as the reference's len()
                keep = sch.last_keep_idx[:kept].long()
                # the scores travel with their rows (the reference leaves them behind, :422-423)
                sch.attention_accumulator[:kept] = sch.attention_accumulator[keep]
                sch.access_timestamps[:kept] = sch.access_timestamps[keep]
                sch.attention_accumulator[kept:cur] = 0
                sch.access_timestamps[kept:cur] = 0
            else:
                # the other policies only evict when the cache is over its size, which the manager never lets
                # happen (:404-410 hand them at most cache_size rows): their mask is empty here
                keep = torch.nonzero(~evict, as_tuple=True)[0]
                kept = int(keep.numel())
            self.cache_keys[:kept] = self.cache_keys[keep]
            self.cache_values[:kept] = self.cache_values[keep]
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
