"""Import aliases with the reference's module paths.

The reference's callers write `from core.single.pikv_routing import TopKBalancedRouter`,
`from core.single.module.pikv_compression import QuantizedCompressor` and so on.  install() registers
this package's modules under those names in sys.modules, so such code runs unchanged on the CUDA
kernels:

    import pikv_b200.compat; pikv_b200.compat.install()
    from core.single.pikv_moe import PiKVMoE

Nothing is registered if a real `core` package is already imported (the reference itself), unless
force=True.
"""
from __future__ import annotations

import importlib
import sys
import types

# reference module path -> module of this package with the same class names and constructors
ALIASES = {
    "core.single.pikv_routing": "pikv_b200.routing",
    "core.single.routing_strategy": "pikv_b200.routing_strategy",
    "core.single.pikv_compression": "pikv_b200.compression",
    "core.single.kv_cache_compression": "pikv_b200.kv_cache_compression",
    "core.single.cache_scheduling": "pikv_b200.scheduling",
    "core.single.pikv_moe": "pikv_b200.moe",
    "core.single.config": "pikv_b200.config",
    "core.single.module.pikv_routing": "pikv_b200.module.routing",
    "core.single.module.pikv_compression": "pikv_b200.module.compression",
    "core.single.module.pikv_scheduling": "pikv_b200.module.scheduling",
}


def install(force: bool = False) -> list:
    """Register the aliases; returns the names registered."""
    if "core" in sys.modules and not force and not getattr(sys.modules["core"], "__pikv_b200_compat__", False):
        raise ImportError("a package named `core` is already imported; pass force=True to shadow its modules")
    done = []
    for pkg in ("core", "core.single", "core.single.module"):
        if pkg not in sys.modules or force:
            m = types.ModuleType(pkg)
            m.__path__ = []                     # a package, so that `import core.single.x` resolves via sys.modules
            m.__pikv_b200_compat__ = True
            sys.modules[pkg] = m
    for name, target in ALIASES.items():
        mod = importlib.import_module(target)
        sys.modules[name] = mod
        parent, _, leaf = name.rpartition(".")
        setattr(sys.modules[parent], leaf, mod)
        done.append(name)
    sys.modules["core"].single = sys.modules["core.single"]
    sys.modules["core.single"].module = sys.modules["core.single.module"]
    for leaf in ("BaseRouter", "TopKBalancedRouter", "AdaptiveRouter", "PiKVRouter", "PyramidCompressor", "SVDCompressor",
                 "QuantizedCompressor", "H2OScheduler"):
        src = importlib.import_module("pikv_b200.module")
        if hasattr(src, leaf):
            setattr(sys.modules["core.single.module"], leaf, getattr(src, leaf))
    return done
