"""PiKVMoE with the constructor, forward and state-dict keys of core/single/pikv_moe.py.

The embedding, the LoRA experts and the vocabulary projection are plain torch modules (they are
outside the routed KV-cache path); the router tail, the cache compressor and the H2O-scheduled cache
manager run on the CUDA kernels.  Parameters are created in the reference's order, so a model built
after torch.manual_seed(s) has the reference's weights for the same seed.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import config
from .kv_cache_compression import KVCacheCompressor
from .routing_strategy import AdaptiveRouter
from .scheduling import CacheSchedulingManager, SchedulingPolicy


class LoRALayer(nn.Module):
    """x @ A @ B * alpha / rank (core/single/lora.py:8-29); A Kaiming-uniform, B zero."""

    def __init__(self, in_features, out_features, rank=4, alpha=1.0, dropout=0.0):
        super().__init__()
        self.rank, self.alpha, self.scaling = rank, alpha, alpha / rank
        self.lora_A = nn.Parameter(torch.zeros(in_features, rank))
        self.lora_B = nn.Parameter(torch.zeros(rank, out_features))
        self.dropout = nn.Dropout(p=dropout)
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B)

    def forward(self, x):
        return self.dropout(x @ self.lora_A @ self.lora_B) * self.scaling


class LoRAExpert(nn.Module):
    """relu(dense(x) + lora(x)) (core/single/lora.py:31-52)."""

    def __init__(self, hidden_size, rank=4, alpha=1.0):
        super().__init__()
        self.hidden_size = hidden_size
        self.dense = nn.Linear(hidden_size, hidden_size)
        self.lora = LoRALayer(hidden_size, hidden_size, rank=rank, alpha=alpha)

    def forward(self, x):
        return F.relu(self.dense(x) + self.lora(x))


class KVCache(nn.Module):
    """core/single/pikv_moe.py:13-137: one mean vector per forward, ring slot or scheduled manager."""

    def __init__(self, size, use_scheduling=False, scheduling_policy=SchedulingPolicy.NONE):
        super().__init__()
        self.size, self.hidden_size, self.use_scheduling = size, config["hidden_size"], use_scheduling
        self.register_buffer("keys", torch.zeros(size, self.hidden_size))
        self.register_buffer("values", torch.zeros(size, self.hidden_size))
        self.register_buffer("importance", torch.zeros(size))
        self.compressor = KVCacheCompressor(hidden_size=self.hidden_size, compression_type="pyramid", compression_ratio=0.5)
        self.value_lora = LoRALayer(self.hidden_size, self.hidden_size, rank=4, alpha=1.0)
        self.scheduling_manager = (CacheSchedulingManager(size, self.hidden_size, scheduling_policy)
                                   if use_scheduling else None)

    def update(self, idx, key, value, importance):
        if key.dim() == 3:
            key, value = key.mean(dim=0).mean(dim=0), value.mean(dim=0).mean(dim=0)
        elif key.dim() == 2:
            key, value = key.mean(dim=0), value.mean(dim=0)
        if self.use_scheduling and self.scheduling_manager is not None:
            self.scheduling_manager.update_cache(key[None, None], value[None, None], {"importance": importance})
        else:
            self.keys[idx] = key
            self.values[idx] = value
            self.importance[idx] = importance.mean()

    def get_all(self):
        if self.use_scheduling and self.scheduling_manager is not None:
            n = self.scheduling_manager._size()
            if n == 0:
                return torch.zeros(self.hidden_size, device=self.keys.device)
            k, v = self.scheduling_manager.cache_keys[:n], self.scheduling_manager.cache_values[:n]
            imp = torch.ones(1, n, device=k.device)
        else:
            k, v, imp = self.keys, self.values, self.importance.unsqueeze(0)
        _, cv = self.compressor(k.unsqueeze(0), v.unsqueeze(0), imp)
        cv = cv + self.value_lora(cv)
        return cv.squeeze(0).mean(dim=0)

    def set_all(self, data):
        """core/single/pikv_moe.py:115-121: a scheduled cache is emptied, a ring cache gets `data` in every slot."""
        if data is None:
            return
        if self.use_scheduling and self.scheduling_manager is not None:
            self.scheduling_manager.reset_cache()
        else:
            self.values.copy_(data.unsqueeze(0).expand(self.size, -1))

    def get_cache_stats(self):
        if self.use_scheduling and self.scheduling_manager is not None:
            return self.scheduling_manager.get_cache_stats()
        return {"cache_size": self.size, "cache_utilization": 1.0, "policy": "none"}

    def change_scheduling_policy(self, new_policy: SchedulingPolicy):
        if self.use_scheduling and self.scheduling_manager is not None:
            self.scheduling_manager.change_policy(new_policy)


class PiKVMoE(nn.Module):
    """core/single/pikv_moe.py:139-336."""

    def __init__(self, rank=4, alpha=1.0, use_distillation=False, teacher_hidden_size=None,
                 use_cache_scheduling=False, cache_scheduling_policy=SchedulingPolicy.NONE):
        super().__init__()
        if use_distillation:
            raise NotImplementedError("distillation is a training aid outside the routed KV-cache path")
        self.use_distillation = False
        self.use_cache_scheduling = use_cache_scheduling
        self.cache_scheduling_policy = cache_scheduling_policy
        h, E = config["hidden_size"], config["num_experts"]
        self.embedding = nn.Embedding(config["vocab_size"], h)
        self.experts = nn.ModuleList([LoRAExpert(h, rank=rank, alpha=alpha) for _ in range(E)])
        self.router = AdaptiveRouter(hidden_size=h, num_experts=E, top_k=2, temperature=1.0)
        self.query_proj = nn.Linear(h, h)
        self.key_proj = nn.Linear(h, h)
        self.query_lora = LoRALayer(h, h, rank=rank, alpha=alpha)
        self.key_lora = LoRALayer(h, h, rank=rank, alpha=alpha)
        self.cache_sizes = self.pyramidal_cache_allocation()
        self.kv_caches = nn.ModuleList([KVCache(size, use_scheduling=use_cache_scheduling,
                                                scheduling_policy=cache_scheduling_policy) for size in self.cache_sizes])
        self.register_buffer("cache_ptrs", torch.zeros(E, dtype=torch.long))
        self.vocab_proj = nn.Linear(h, config["vocab_size"])
        self._host_ptrs = None

    def pyramidal_cache_allocation(self):
        c1, d = config["kv_cache_size"], config["cache_decrement"]
        return [c1 - (i - 1) * d for i in range(1, config["num_layers"] + 1)]

    def compute_token_importance(self, query, key):
        q = self.query_proj(query) + self.query_lora(query)
        k = self.key_proj(key) + self.key_lora(key)
        scores = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(config["hidden_size"])
        return F.softmax(scores, dim=-1).sum(dim=1)

    def update_cache(self, expert_idx, key, value, importance):
        cache = self.kv_caches[expert_idx]
        if self._host_ptrs is None:
            self._host_ptrs = self.cache_ptrs.tolist()
        ptr = self._host_ptrs[expert_idx]
        cache.update(ptr, key, value, importance)
        if not self.use_cache_scheduling:
            self._host_ptrs[expert_idx] = (ptr + 1) % cache.size
            self.cache_ptrs[expert_idx] = self._host_ptrs[expert_idx]

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self._host_ptrs = None          # the ring pointers are read again from the loaded cache_ptrs

    # -- cache scheduling switches, core/single/pikv_moe.py:338-379 -------------------------------------
    def enable_cache_scheduling(self, policy: SchedulingPolicy = SchedulingPolicy.LRU):
        self.use_cache_scheduling, self.cache_scheduling_policy = True, policy
        for cache in self.kv_caches:
            cache.use_scheduling = True
            if cache.scheduling_manager is None:
                cache.scheduling_manager = CacheSchedulingManager(cache.size, cache.hidden_size, policy).to(cache.keys.device)
            else:
                cache.scheduling_manager.change_policy(policy)

    def disable_cache_scheduling(self):
        self.use_cache_scheduling = False
        for cache in self.kv_caches:
            cache.use_scheduling = False
            if cache.scheduling_manager is not None:
                cache.scheduling_manager.reset_cache()

    def change_cache_scheduling_policy(self, new_policy: SchedulingPolicy):
        if self.use_cache_scheduling:
            self.cache_scheduling_policy = new_policy
            for cache in self.kv_caches:
                cache.change_scheduling_policy(new_policy)

    def get_cache_stats(self):
        return {f"expert_{i}": cache.get_cache_stats() for i, cache in enumerate(self.kv_caches)}

    # -- checkpoints, core/single/pikv_moe.py:456-505 -----------------------------------------------------
    def save_checkpoint(self, path):
        """The reference's dictionary (same keys).  `model_state_dict` already holds every cache buffer
        (ring slots or the scheduled manager's rows and scores), so a load restores the caches exactly;
        `kv_caches` (one mean vector per cache) is written as the reference writes it."""
        checkpoint = {
            "model_state_dict": self.state_dict(),
            "cache_ptrs": self.cache_ptrs,
            "kv_caches": [cache.get_all() for cache in self.kv_caches],
            "use_distillation": self.use_distillation,
            "use_cache_scheduling": self.use_cache_scheduling,
            "cache_scheduling_policy": self.cache_scheduling_policy.value if self.use_cache_scheduling else None,
        }
        if self.use_cache_scheduling:
            checkpoint["cache_stats"] = self.get_cache_stats()
        torch.save(checkpoint, path)

    def load_checkpoint(self, path):
        """Inverse of save_checkpoint, in the reference's order: state dict, ring pointers, then set_all with
        the saved mean vectors (which, as in the reference, overwrites a ring cache's value rows with that
        vector and empties a scheduled cache), then the scheduling settings."""
        checkpoint = torch.load(path, map_location=self.cache_ptrs.device, weights_only=False)
        self.load_state_dict(checkpoint["model_state_dict"])
        self.cache_ptrs.copy_(checkpoint["cache_ptrs"])
        self._host_ptrs = None
        for i, data in enumerate(checkpoint["kv_caches"]):
            if data is not None:
                self.kv_caches[i].set_all(data)
        if checkpoint.get("use_cache_scheduling", False):
            try:
                self.enable_cache_scheduling(SchedulingPolicy(checkpoint.get("cache_scheduling_policy", "none")))
            except ValueError:
                pass

    def forward(self, x, query=None, return_loss=False, targets=None, use_teacher=False):
        if x.dim() == 2:
            x = self.embedding(x)
        elif x.dim() != 3:
            raise ValueError(f"Input must be 2D (token IDs) or 3D (embeddings), got shape: {x.shape}")
        if x.dtype != torch.float32:
            x = x.to(torch.float32)
        routing_weights, expert_indices, top_k_weights, lb_loss, importance = self.router(x)
        if query is not None:
            importance = self.compute_token_importance(query.to(torch.float32), x)
        out = torch.zeros_like(x)
        for i, expert in enumerate(self.experts):
            y = expert(x)
            cached = self.kv_caches[i].get_all()
            if cached is not None:
                y = y + cached[None, None]
            self.update_cache(i, x.detach(), y.detach(), importance.detach())
            out = out + y * routing_weights[:, :, i].unsqueeze(-1)
        logits = self.vocab_proj(out)
        if return_loss:
            return logits, lb_loss
        return logits
