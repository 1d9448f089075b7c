"""Operator variants with the surface of core/single/module/*.py."""
from .compression import BaseCompressor, PyramidCompressor, SVDCompressor, QuantizedCompressor  # noqa: F401
from .routing import BaseRouter, TopKBalancedRouter, AdaptiveRouter, PiKVRouter  # noqa: F401
from .scheduling import H2OScheduler, AdaKVScheduler, DuoAttentionScheduler  # noqa: F401
