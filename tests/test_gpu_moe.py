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


@pytest.mark.parametrize("tag", ["plain", "h2o"])
def test_pikv_moe_checkpoint_round_trip(tag, tmp_path):
    """save_checkpoint / load_checkpoint (core/single/pikv_moe.py:456-505): a model restored into an instance
    that has already stepped continues exactly like a fresh instance restored from the same file (the ring
    pointers are re-read from the loaded state, not kept from before the load)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from pikv_b200.moe import PiKVMoE
    from pikv_b200.scheduling import SchedulingPolicy
    kw = dict(use_cache_scheduling=True, cache_scheduling_policy=SchedulingPolicy.H2O) if tag == "h2o" else {}
    torch.manual_seed(0)
    m = PiKVMoE(**kw).eval().cuda()
    gen = torch.Generator().manual_seed(5)
    xs = [torch.randn(4, 32, 256, generator=gen).cuda() for _ in range(3)]
    path = str(tmp_path / "ckpt.pt")
    with torch.no_grad():
        m(xs[0])
        m.save_checkpoint(path)
        ckpt = torch.load(path, weights_only=False)
        assert set(ckpt) >= {"model_state_dict", "cache_ptrs", "kv_caches", "use_distillation", "use_cache_scheduling",
                             "cache_scheduling_policy"}
        assert ckpt["cache_scheduling_policy"] == ("h2o" if tag == "h2o" else None)
        m(xs[1])                                   # moves the ring pointers / caches past the saved state
        m.load_checkpoint(path)
        got = m(xs[2])
        torch.manual_seed(123)                     # other initial weights: everything must come from the file
        fresh = PiKVMoE(**kw).eval().cuda()
        fresh.load_checkpoint(path)
        want = fresh(xs[2])
    assert torch.equal(m.cache_ptrs, fresh.cache_ptrs)
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)
    assert set(m.get_cache_stats()) == {f"expert_{i}" for i in range(len(m.kv_caches))}
