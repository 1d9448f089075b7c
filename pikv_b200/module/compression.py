"""Compressors with the surface of core/single/module/pikv_compression.py (the variant with
symmetric quantisation and a working adaptive SVD rank)."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..compression import _linear


class BaseCompressor(nn.Module):
    """core/single/module/pikv_compression.py:38-104."""

    def __init__(self, hidden_size: int, compression_ratio: float = 0.5):
        super().__init__()
        self.hidden_size = hidden_size
        self.compression_ratio = compression_ratio
        self.register_buffer("total_original_size", torch.tensor(0.0))
        self.register_buffer("total_compressed_size", torch.tensor(0.0))
        self.register_buffer("compression_count", torch.tensor(0.0))

    def forward(self, keys, values, importance=None):
        self._update_stats(keys.numel(), keys.numel())
        return keys, values

    def get_compression_stats(self) -> Dict[str, float]:
        tot = self.total_original_size.item()
        actual = self.total_compressed_size.item() / tot if tot > 0 else 1.0
        return {"target_compression_ratio": self.compression_ratio, "actual_compression_ratio": actual,
                "memory_reduction": 1.0 - actual, "compression_count": self.compression_count.item()}

    def _update_stats(self, original_size: int, compressed_size: int):
        self.total_original_size += original_size
        self.total_compressed_size += compressed_size
        self.compression_count += 1

    def reset_stats(self):
        self.total_original_size.zero_()
        self.total_compressed_size.zero_()
        self.compression_count.zero_()


class PyramidCompressor(BaseCompressor):
    """core/single/module/pikv_compression.py:106-260: per level an encoder (Linear, LayerNorm, ReLU) and a
    decoder (Linear, LayerNorm); a token of level L runs encoders 0..L, decoders L..0 and adds the result
    to itself.  Levels come from importance thresholds linspace(0.8, 0.2, num_levels)."""

    def __init__(self, hidden_size: int, compression_ratio: float = 0.5, num_levels: int = 3, decay_factor: float = 0.8,
                 use_adaptive_levels: bool = True):
        super().__init__(hidden_size, compression_ratio)
        self.num_levels = num_levels
        self.decay_factor = decay_factor
        self.use_adaptive_levels = use_adaptive_levels
        self.compression_layers = nn.ModuleList()
        size, ratio = hidden_size, compression_ratio
        for _ in range(num_levels):
            out = max(int(size * ratio), 1)
            self.compression_layers.append(nn.ModuleDict({
                "encoder": nn.Sequential(nn.Linear(size, out), nn.LayerNorm(out), nn.ReLU()),
                "decoder": nn.Sequential(nn.Linear(out, size), nn.LayerNorm(size)),
            }))
            size, ratio = out, ratio * decay_factor
        self.register_buffer("importance_thresholds", torch.linspace(0.8, 0.2, num_levels))
        for layer in self.compression_layers:
            for seq in layer.values():
                for m in seq:
                    if isinstance(m, nn.Linear):
                        nn.init.xavier_normal_(m.weight)
                        nn.init.zeros_(m.bias)

    def _assign_compression_levels(self, importance: torch.Tensor) -> torch.Tensor:
        """:167-184.  Level 0 marks "not assigned yet" in the reference's loop, so a token gets the first level
        L >= 1 (below the last) whose threshold it reaches, and the last level otherwise; with one level
        everything stays at 0."""
        levels = torch.full_like(importance, self.num_levels - 1, dtype=torch.long)
        for level in range(self.num_levels - 2, 0, -1):
            levels = torch.where(importance >= self.importance_thresholds[level], torch.full_like(levels, level), levels)
        return levels

    def _chain(self, x: torch.Tensor, level: int) -> torch.Tensor:
        y = x
        for i in range(level + 1):
            enc = self.compression_layers[i]["encoder"]
            y = torch.relu(enc[1](_linear(enc[0], y, relu=False)))
        for i in range(level, -1, -1):
            dec = self.compression_layers[i]["decoder"]
            y = dec[1](_linear(dec[0], y, relu=False))
        return x + y

    def _apply_pyramid_compression(self, x: torch.Tensor, levels: torch.Tensor) -> torch.Tensor:
        out = torch.zeros_like(x)
        for level in range(self.num_levels):
            mask = levels == level
            idx = mask.reshape(-1).nonzero(as_tuple=True)[0]
            if idx.numel() == 0:
                continue
            flat = x.reshape(-1, x.shape[-1])
            out.view(-1, x.shape[-1])[idx] = self._chain(flat[idx], level)
        return out

    def forward(self, keys: torch.Tensor, values: torch.Tensor, importance: Optional[torch.Tensor] = None):
        b, s, _ = keys.shape
        if importance is None:
            importance = torch.full((b, s), 0.5, device=keys.device)
        levels = self._assign_compression_levels(importance)
        ck = self._apply_pyramid_compression(keys, levels)
        cv = self._apply_pyramid_compression(values, levels)
        original = keys.numel() + values.numel()
        share = torch.bincount(levels.reshape(-1), minlength=self.num_levels).float() / levels.numel()
        avg = sum((self.decay_factor ** lv) * float(share[lv]) for lv in range(self.num_levels))
        self._update_stats(original, int(original * avg))
        return ck, cv


class QuantizedCompressor(BaseCompressor):
    """core/single/module/pikv_compression.py:918-1060."""

    def __init__(self, hidden_size: int, bits: int = 8, group_size: int = 128, symmetric: bool = False,
                 dynamic: bool = True):
        super().__init__(hidden_size, bits / 32)
        self.bits = bits
        self.group_size = min(group_size, hidden_size)
        self.symmetric = symmetric
        self.dynamic = dynamic
        self.register_buffer("scale", torch.ones(1))
        self.register_buffer("zero_point", torch.zeros(1))
        self.register_buffer("quantization_error", torch.zeros(1))
        self.calibrated = False

    def _qrange(self) -> Tuple[int, int]:
        # :947-963 - the signed range exists for 4, 8 and 16 bits only
        if self.symmetric and self.bits in (4, 8, 16):
            return -(1 << (self.bits - 1)), (1 << (self.bits - 1)) - 1
        return 0, 2 ** self.bits - 1

    def _static_params(self, first_block: torch.Tensor, groups: int) -> torch.Tensor:
        if not self.calibrated:
            qmin, qmax = self._qrange()
            _, _, p, _ = ops.quant_block(first_block.contiguous(), self.group_size, qmin, qmax, self.symmetric,
                                         want_err=False)
            self.scale, self.zero_point = p[0, 0].clone(), p[0, 1].clone()
            self.calibrated = True
        return torch.stack([self.scale.reshape(()), self.zero_point.reshape(())]).float().repeat(groups, 1).contiguous()

    def forward(self, keys: torch.Tensor, values: torch.Tensor, importance: Optional[torch.Tensor] = None):
        shape = keys.shape
        kf, vf = keys.reshape(-1, shape[-1]), values.reshape(-1, shape[-1])
        groups = (shape[-1] + self.group_size - 1) // self.group_size
        qmin, qmax = self._qrange()
        params_in = None if self.dynamic else self._static_params(kf[:, : self.group_size], groups)
        dk, _, _, _ = ops.quant_block(kf, self.group_size, qmin, qmax, self.symmetric, params_in=params_in)
        dv, _, _, err = ops.quant_block(vf, self.group_size, qmin, qmax, self.symmetric, params_in=params_in)
        with torch.no_grad():
            last_w = shape[-1] - (groups - 1) * self.group_size
            self.quantization_error = err[-1] / float(vf.shape[0] * last_w)
        original = keys.numel() + values.numel()
        self._update_stats(original, int(original * self.bits / 32))
        return dk.to(keys.dtype).reshape(shape), dv.to(values.dtype).reshape(shape)

    def get_compression_stats(self) -> Dict[str, float]:
        stats = super().get_compression_stats()
        stats.update({"bits": self.bits, "quantization_error": float(self.quantization_error),
                      "group_size": self.group_size})
        return stats


class SVDCompressor(BaseCompressor):
    """core/single/module/pikv_compression.py:788-916: latent columns beyond the adaptive rank are
    zeroed before the reconstruction."""

    def __init__(self, hidden_size: int, rank: Optional[int] = None, compression_ratio: float = 0.5,
                 adaptive_rank: bool = True, energy_threshold: float = 0.95):
        super().__init__(hidden_size, compression_ratio)
        self.rank = rank or int(hidden_size * compression_ratio)
        self.adaptive_rank = adaptive_rank
        self.energy_threshold = energy_threshold
        self.key_projector = nn.Linear(hidden_size, self.rank)
        self.key_reconstructor = nn.Linear(self.rank, hidden_size)
        self.value_projector = nn.Linear(hidden_size, self.rank)
        self.value_reconstructor = nn.Linear(self.rank, hidden_size)
        self.register_buffer("effective_rank", torch.tensor(float(self.rank)))
        self.register_buffer("energy_preserved", torch.tensor(0.0))
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.orthogonal_(m.weight)
                nn.init.zeros_(m.bias)

    def _compute_adaptive_rank(self, x: torch.Tensor) -> int:
        """:827-862 - eigenvalues of the covariance, smallest rank reaching the energy threshold."""
        if not self.adaptive_rank:
            return self.rank
        try:
            flat = x.reshape(-1, x.size(-1)).float()
            cov = torch.mm(flat.t(), flat) / flat.size(0)
            ev = torch.linalg.eigh(cov)[0].flip(0)
            ratios = torch.cumsum(ev, dim=0) / torch.sum(ev)
            below = ratios < self.energy_threshold
            eff = int(below.sum().item()) + 1 if below.any() else 1
            self.effective_rank = torch.tensor(float(eff), device=x.device)
            self.energy_preserved = ratios[min(eff - 1, len(ratios) - 1)]
            return max(eff, 1)
        except Exception:
            return self.rank

    def _one(self, x, proj, rec, r):
        z = _linear(proj, x, False)
        if r < self.rank:
            z = torch.cat([z[..., :r], torch.zeros_like(z[..., r:])], dim=-1)
        return _linear(rec, torch.relu(z), False)

    def forward(self, keys: torch.Tensor, values: torch.Tensor, importance: Optional[torch.Tensor] = None):
        r = self._compute_adaptive_rank(keys)
        rk = self._one(keys, self.key_projector, self.key_reconstructor, r)
        rv = self._one(values, self.value_projector, self.value_reconstructor, r)
        original = keys.numel() + values.numel()
        self._update_stats(original, int(original * r / self.hidden_size))
        return rk, rv

    def get_compression_stats(self) -> Dict[str, float]:
        stats = super().get_compression_stats()
        stats.update({"effective_rank": self.effective_rank.item(), "energy_preserved": self.energy_preserved.item(),
                      "adaptive_rank": self.adaptive_rank, "rank": self.rank})
        return stats
