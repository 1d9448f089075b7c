"""pikv_b200: the routed KV-cache hot path of PiKV as sm_100a CUDA kernels.

Operator classes keep the reference's names and signatures; the kernels sit
behind the C ABI in include/pikv_b200.h (libpikv_b200.so, built by
`python -m pikv_b200.build`).  There is no CPU fallback: using an operator
without the built library, or with CPU tensors, raises PikvError.
"""
from ._lib import PikvError, lib, launch_count  # noqa: F401
from . import ops  # noqa: F401
from .paged_cache import PagedKVCache  # noqa: F401
from .routing import BaseRouter, TopKBalancedRouter, AdaptiveRouter, PiKVRouter  # noqa: F401
from .compression import BaseCompressor, PyramidCompressor, SVDCompressor, QuantizedCompressor  # noqa: F401
from .scheduling import (SchedulingPolicy, H2OScheduler, StreamingLLMScheduler, QUESTScheduler, FlexGenScheduler,  # noqa: F401
                         LRUScheduler, LRUPlusScheduler, CacheSchedulingManager)

__all__ = [
    "PikvError", "lib", "launch_count", "ops", "PagedKVCache",
    "BaseRouter", "TopKBalancedRouter", "AdaptiveRouter", "PiKVRouter",
    "BaseCompressor", "PyramidCompressor", "SVDCompressor", "QuantizedCompressor",
    "SchedulingPolicy", "H2OScheduler", "StreamingLLMScheduler", "QUESTScheduler", "FlexGenScheduler", "LRUScheduler",
    "LRUPlusScheduler", "CacheSchedulingManager",
]
