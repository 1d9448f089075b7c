"""The compressor inside PiKVMoE's KVCache, surface of core/single/kv_cache_compression.py."""
from __future__ import annotations

import torch
import torch.nn as nn

from .compression import _linear


class PyramidCompression(nn.Module):
    """core/single/kv_cache_compression.py:6-45: xi = x * importance; xi + L(h/2, h)(L(h, h/2)(xi)).
    bf16 inputs take the tcgen05 projection kernel, fp32 inputs cuBLAS."""

    def __init__(self, hidden_size, compression_ratio=0.5):
        super().__init__()
        self.hidden_size, self.compression_ratio = hidden_size, compression_ratio
        mid = int(hidden_size * compression_ratio)
        self.compression_layers = nn.ModuleList([nn.Linear(hidden_size, mid), nn.Linear(mid, hidden_size)])
        self.importance_weights = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x, importance=None):
        if importance is not None:
            x = x * importance.unsqueeze(-1)
        return x + _linear(self.compression_layers[1], _linear(self.compression_layers[0], x, False), False)


class KVCacheCompressor(nn.Module):
    """core/single/kv_cache_compression.py:101-127 ('pyramid' only; 'dynamic' is outside the routed path)."""

    def __init__(self, hidden_size, compression_type="pyramid", **kwargs):
        super().__init__()
        self.hidden_size = hidden_size
        if compression_type != "pyramid":
            raise ValueError(f"compression type {compression_type!r} is not served by pikv_b200")
        self.compressor = PyramidCompression(hidden_size, **kwargs)

    def forward(self, keys, values, importance=None):
        return self.compressor(keys, importance), self.compressor(values, importance)
