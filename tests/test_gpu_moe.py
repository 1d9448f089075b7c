"""Config 1 end to end: PiKVMoE [8,128,256] fp32, 4 experts top-2, against the reference's logits."""
import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tag", ["plain", "h2o"])
def test_pikv_moe_matches_reference_logits(tag):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import pikv_b200
    from pikv_b200.moe import PiKVMoE
    from pikv_b200.scheduling import SchedulingPolicy
    g = load_golden("pikv_moe_c1")
    kw = dict(use_cache_scheduling=True, cache_scheduling_policy=SchedulingPolicy.H2O) if tag == "h2o" else {}
    torch.manual_seed(0)                       # same seed, same construction order: the reference's weights
    m = PiKVMoE(**kw).eval().cuda()
    gen = torch.Generator().manual_seed(1)
    before = pikv_b200.launch_count()
    with torch.no_grad():
        for step in range(2):                  # the second forward reads what the first one cached
            x = torch.randn(8, 128, 256, generator=gen).cuda()
            logits = m(x)
            ref_head, ref_stride = g[f"{tag}/logits_head{step}"], g[f"{tag}/logits_stride{step}"]
            scale = float(g[f"{tag}/logits_absmax{step}"])
            assert np.abs(logits[:, :, :48].cpu().numpy() - ref_head).max() <= 1e-5 * scale
            assert np.abs(logits[:, ::16, ::997].cpu().numpy() - ref_stride).max() <= 1e-5 * scale
            assert abs(float(logits.abs().max()) - scale) <= 1e-5 * scale
    assert pikv_b200.launch_count() - before >= 12          # the router tails ran on the CUDA kernels
    np.testing.assert_array_equal(m.cache_ptrs.cpu().numpy(), g[f"{tag}/cache_ptrs"])
