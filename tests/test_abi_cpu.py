"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from pikv_b200 import build
    path = build.build()
    assert os.path.exists(path)
    return ctypes.CDLL(path)


def header_symbols():
    text = open(os.path.join(ROOT, "include", "pikv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pikv_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(built_lib):
    names = header_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(built_lib, n), f"{n} declared in include/pikv_b200.h but not exported"


def test_binding_table_matches_header():
    from pikv_b200 import _lib
    assert sorted(_lib.SIGNATURES) == header_symbols()


def test_version_and_pure_host_entry_points(built_lib):
    from pikv_b200 import _lib
    lib = _lib.lib()
    assert lib.pikv_abi_version() == _lib.ABI_VERSION
    assert lib.pikv_gate_workspace_bytes(16384, 8, 2) > 0
    assert lib.pikv_quant_block_workspace_bytes(1024, 256, 1) > 0
    # 16 header + K,V codes + scales, rounded to 16 bytes
    assert lib.pikv_a2a_record_bytes(8) == 16 + 2 * 8 * 128 + 4 * 8
    # the page prefix of the streams + one partial (128 outputs, max, denominator) per (worker group + stream, query head)
    ws = lib.pikv_decode_attn_workspace_bytes(64, 32, 8, 32768, 8)
    assert ws >= 65 * 4 + 64 * 32 * 130 * 4 and ws % 4 == 0
    assert lib.pikv_decode_attn_workspace_bytes(128, 32, 8, 32768, 0) > ws
    assert lib.pikv_shard_decode_buffer_bytes(0, 8, 256, 2, 32) == 256 * 32 * 128 * 2


def test_argument_errors_are_reported_without_a_gpu(built_lib):
    from pikv_b200 import _lib
    lib = _lib.lib()
    p = _lib.GateParams()
    assert lib.pikv_gate_fused(ctypes.byref(p), None) == -1          # PIKV_EINVAL: T, E, top_k = 0
    assert b"positive" in lib.pikv_last_error()
    p.T, p.E, p.top_k = 4, 100, 2
    assert lib.pikv_gate_fused(ctypes.byref(p), None) == -4          # PIKV_ELIMIT: E > 64
    a = _lib.AppendParams()
    a.T, a.n_kv, a.top_k = 4, 8, 2
    assert lib.pikv_kv_append_quant(ctypes.byref(a), None) == -1
    assert lib.pikv_lowrank_project(None, None, None, None, None, 1, 128, 64, 1024, 1, None) == -1


def test_operators_refuse_cpu_tensors(built_lib):
    import torch
    import pikv_b200
    with pytest.raises(pikv_b200.PikvError):
        pikv_b200.ops.gate_fused(logits=torch.randn(4, 8), top_k=2)
    r = pikv_b200.TopKBalancedRouter(32, 4)
    with pytest.raises(pikv_b200.PikvError):
        r(torch.randn(1, 4, 32))


def test_pikv_moe_builds_with_the_reference_weights_for_a_seed():
    """Same constructor order as core/single/pikv_moe.py: after manual_seed(0) the drop-in holds the
    reference's parameters (count and sum recorded by the fixture generator).  No GPU involved."""
    import numpy as np
    import torch
    from conftest import load_golden
    from pikv_b200.moe import PiKVMoE
    from pikv_b200.scheduling import SchedulingPolicy
    g = load_golden("pikv_moe_c1")
    for tag, kw in (("plain", {}), ("h2o", dict(use_cache_scheduling=True, cache_scheduling_policy=SchedulingPolicy.H2O))):
        torch.manual_seed(0)
        m = PiKVMoE(**kw)
        assert sum(p.numel() for p in m.parameters()) == int(g[f"{tag}/n_params"])
        assert abs(sum(p.double().sum().item() for p in m.parameters()) - float(g[f"{tag}/param_sum"])) < 1e-6


def test_reference_import_paths_resolve():
    """pikv_b200.compat.install() makes the reference's own import lines work on this package's classes."""
    import subprocess
    import sys
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import pikv_b200.compat as c; c.install()\n"
        "from core.single.pikv_routing import BaseRouter, TopKBalancedRouter, PiKVRouter\n"
        "from core.single.pikv_compression import QuantizedCompressor, PyramidCompressor, SVDCompressor\n"
        "from core.single.cache_scheduling import H2OScheduler, CacheSchedulingManager, SchedulingPolicy\n"
        "from core.single.module.pikv_scheduling import AdaKVScheduler, DuoAttentionScheduler\n"
        "from core.single.module import QuantizedCompressor as MQ\n"
        "from core.single.pikv_moe import PiKVMoE\n"
        "import pikv_b200\n"
        "assert TopKBalancedRouter is pikv_b200.TopKBalancedRouter and PiKVMoE.__module__ == 'pikv_b200.moe'\n"
    ) % ROOT
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
