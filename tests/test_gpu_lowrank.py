"""GPU parity: the tcgen05 projection kernel and the SVD / Pyramid compressors against the
oracle and the reference's golden vectors.  bf16 tensor-core outputs: 1e-2 relative;
fp32 module outputs: 1e-5."""
import numpy as np
import pytest
import torch

from conftest import load_golden, sub
from oracle import pikv_oracle as O

pytestmark = pytest.mark.gpu
F32 = np.float32


@pytest.fixture(autouse=True)
def _no_grad():
    with torch.no_grad():
        yield


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-12)


def state(dev, weights):
    return {k: torch.from_numpy(np.array(v)).to(dev) for k, v in weights.items()}


@pytest.mark.parametrize("M,N,K,relu", [(128, 64, 64, True), (128, 64, 1024, True), (1000, 32, 1024, True),
                                        (4096, 16, 1024, False), (300, 1024, 64, False), (700, 1024, 32, False), (260, 256, 16, True), (513, 256, 128, True),
                                        (8192, 64, 1024, True)])
def test_lowrank_project_matches_oracle(dev, M, N, K, relu):
    import pikv_b200
    from pikv_b200 import ops
    torch.manual_seed(M + N)
    x = torch.randn(M, K).bfloat16()
    w = torch.nn.init.orthogonal_(torch.empty(max(N, K), max(N, K)))[:N, :K].contiguous().bfloat16()
    b = torch.randn(N) * 0.1
    y = ops.lowrank_project(x.to(dev), w.to(dev), b.to(dev), relu=relu, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert pikv_b200.lib().pikv_lowrank_error_state() == 0
    want = x.float().numpy() @ w.float().numpy().T + b.numpy()
    if relu:
        want = np.maximum(want, 0)
    # operands are exact bf16, products exact in fp32: only the accumulation order differs
    assert rel(y.cpu().numpy(), want) < 1e-4
    yb = ops.lowrank_project(x.to(dev), w.to(dev), b.to(dev), relu=relu, out_dtype=torch.bfloat16)
    assert rel(yb.float().cpu().numpy(), want) < 1e-2
    res = torch.randn(M, N).bfloat16()
    yr = ops.lowrank_project(x.to(dev), w.to(dev), b.to(dev), relu=relu, residual=res.to(dev), out_dtype=torch.float32)
    assert rel(yr.cpu().numpy(), want + res.float().numpy()) < 1e-4


def test_svd_compressor_fp32_matches_reference(dev):
    import pikv_b200
    g = load_golden("lowrank_svd_single")
    c = pikv_b200.SVDCompressor(64, rank=16).to(dev)
    c.load_state_dict(state(dev, sub(g, "weights")))
    rk, rv = c(torch.from_numpy(g["keys"]).to(dev), torch.from_numpy(g["values"]).to(dev))
    assert rel(rk.cpu().numpy(), g["rec_keys"]) < 1e-5
    assert rel(rv.cpu().numpy(), g["rec_values"]) < 1e-5


def test_svd_compressor_module_adaptive_rank_matches_reference(dev):
    from pikv_b200.module import SVDCompressor
    g = load_golden("lowrank_svd_module")
    c = SVDCompressor(64, rank=16, adaptive_rank=True, energy_threshold=0.5).to(dev)
    c.load_state_dict(state(dev, sub(g, "weights")))
    rk, rv = c(torch.from_numpy(g["keys"]).to(dev), torch.from_numpy(g["values"]).to(dev))
    assert float(c.effective_rank) == float(g["effective_rank"])
    assert rel(rk.cpu().numpy(), g["rec_keys"]) < 1e-5
    assert rel(rv.cpu().numpy(), g["rec_values"]) < 1e-5


def test_pyramid_compressor_fp32_matches_reference(dev):
    import pikv_b200
    g = load_golden("pyramid_single")
    c = pikv_b200.PyramidCompressor(64, compression_ratio=0.5, num_levels=3, decay_factor=0.8).to(dev)
    c.load_state_dict(state(dev, sub(g, "weights")))
    k, v = torch.from_numpy(g["keys"]).to(dev), torch.from_numpy(g["values"]).to(dev)
    uk, uv = c(k, v)
    assert rel(uk.cpu().numpy(), g["uni_keys"]) < 1e-5 and rel(uv.cpu().numpy(), g["uni_values"]) < 1e-5
    ik, iv = c(k, v, torch.from_numpy(g["importance"]).to(dev))
    assert rel(ik.cpu().numpy(), g["imp_keys"]) < 1e-5 and rel(iv.cpu().numpy(), g["imp_values"]) < 1e-5


def test_module_pyramid_compressor_matches_reference(dev):
    """core/single/module PyramidCompressor: LayerNorm encoders/decoders, threshold levels, residual."""
    from pikv_b200.module import PyramidCompressor
    g = load_golden("pyramid_module")
    c = PyramidCompressor(64, compression_ratio=0.5, num_levels=3).to(dev)
    c.load_state_dict(state(dev, sub(g, "weights")))
    k, v = torch.from_numpy(g["keys"]).to(dev), torch.from_numpy(g["values"]).to(dev)
    imp = torch.from_numpy(g["importance"]).to(dev)
    np.testing.assert_array_equal(c._assign_compression_levels(imp).cpu().numpy(), g["levels"])
    ck, cv = c(k, v, imp)
    assert rel(ck.cpu().numpy(), g["ck"]) < 1e-5 and rel(cv.cpu().numpy(), g["cv"]) < 1e-5
    nk, nv = c(k, v)
    assert rel(nk.cpu().numpy(), g["nk"]) < 1e-5 and rel(nv.cpu().numpy(), g["nv"]) < 1e-5
    assert float(c.total_compressed_size) == float(g["stats"][0])


def test_svd_compressor_bf16_runs_on_tensor_cores(dev):
    """Config-4 shaped (scaled down): [tokens, 1024] bf16 -> rank 64/32/16 -> 1024, against the fp32 oracle."""
    import pikv_b200
    torch.manual_seed(0)
    x = torch.randn(4, 512, 1024).bfloat16()
    for rank in (64, 32, 16):
        c = pikv_b200.SVDCompressor(1024, rank=rank).to(dev)
        before = pikv_b200.launch_count()
        rk, rv = c(x.to(dev), x.to(dev))
        assert pikv_b200.launch_count() - before == 4          # two projections + two reconstructions, all on the kernel
        w = {k: v.detach().bfloat16().float().cpu().numpy() for k, v in c.state_dict().items()}
        y = O.lowrank_project(x.float().numpy().reshape(-1, 1024), w["key_projector.weight"], w["key_projector.bias"])
        want = O.lowrank_reconstruct(O.bf16_round(y), w["key_reconstructor.weight"], w["key_reconstructor.bias"])
        assert rel(rk.float().cpu().numpy().reshape(-1, 1024), want) < 1e-2
    torch.cuda.synchronize()
    assert pikv_b200.lib().pikv_lowrank_error_state() == 0


def test_full_size_lowrank_matches_oracle(dev):
    """Config 4 at full size: 262144 rows x 1024 -> rank 64 / 32 / 16 on the tensor-core kernel, bf16 out;
    4096 sampled rows (first and last tiles included) against the fp32 oracle at 1e-2."""
    import pikv_b200
    from pikv_b200 import ops
    M, K = 262144, 1024
    g = torch.Generator(device=dev).manual_seed(4)
    x = torch.randn(M, K, generator=g, device=dev).bfloat16()
    rows = np.unique(np.concatenate([np.arange(256), np.arange(M - 256, M),
                                     np.random.default_rng(4).integers(0, M, 3584)]))
    xs = x[torch.from_numpy(rows).to(dev)].float().cpu().numpy()
    for r in (64, 32, 16):
        w = torch.nn.init.orthogonal_(torch.empty(K, K))[:r].contiguous().bfloat16()
        b = torch.randn(r) * 0.05
        y = ops.lowrank_project(x, w.to(dev), b.to(dev), relu=True)
        torch.cuda.synchronize()
        assert pikv_b200.lib().pikv_lowrank_error_state() == 0
        want = O.lowrank_project(xs, w.float().numpy(), b.numpy())
        got = y[torch.from_numpy(rows).to(dev)].float().cpu().numpy()
        assert rel(got, want) < 1e-2, r
