"""GPU parity: the fused gate kernel and the router classes against the oracle and the
reference's golden vectors.  Integer outputs must be bit-exact; probabilities and
weights within 1e-5 relative (fp32)."""
import numpy as np
import pytest
import torch

from conftest import load_golden, sub
from oracle import pikv_oracle as O

pytestmark = pytest.mark.gpu

F32 = np.float32


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-12)


def check_gate(g, logits, k, cap, E, **tail):
    """Everything the kernel derives from given logits must equal the oracle's."""
    probs, idx, tw = O.gate_tail(logits, k, **tail)
    gi = g.topk_idx.cpu().numpy()
    # identical logits -> identical experts, except where two probabilities are closer than fp32 exp noise
    same = (gi == idx).all(axis=1)
    margin = O.topk_margin(probs, k)
    assert (same | (margin < 1e-6)).all(), f"{(~same).sum()} tokens differ beyond the near-tie margin"
    assert rel(g.probs.cpu().numpy(), probs) < 1e-5
    ok = same
    assert rel(g.topk_w.cpu().numpy()[ok], tw[ok]) < 1e-5
    slot, counts_k = O.slot_assign_fast(gi, E, cap if cap > 0 else 1 << 30)
    np.testing.assert_array_equal(g.slot.cpu().numpy(), slot)
    np.testing.assert_array_equal(g.counts_k.cpu().numpy(), counts_k)
    assert rel(g.prob_sum.cpu().numpy(), probs.sum(0)) < 1e-5
    want_len = np.minimum(counts_k.sum(0), cap) if cap > 0 else counts_k.sum(0)
    np.testing.assert_array_equal(g.new_len.cpu().numpy(), want_len)
    return int((~same).sum())


@pytest.mark.parametrize("T,E,k", [(1, 4, 2), (37, 4, 2), (1024, 8, 2), (5000, 64, 2), (777, 16, 4), (300, 64, 8),
                                   (16384, 8, 2)])
def test_gate_from_logits(dev, T, E, k):
    from pikv_b200 import ops
    rng = np.random.default_rng(T + E)
    logits = rng.standard_normal((T, E)).astype(F32) * 2
    cap = O.capacity(T, 1.5, k, E)
    g = ops.gate_fused(logits=torch.from_numpy(logits).to(dev), top_k=k, capacity=cap)
    check_gate(g, logits, k, cap, E)


def test_gate_mask_correction_temperature(dev):
    from pikv_b200 import ops, _lib
    rng = np.random.default_rng(3)
    T, E, k = 2000, 8, 2
    logits = rng.standard_normal((T, E)).astype(F32)
    mask = np.array([1, 1, 0, 1, 1, 0, 1, 1], F32)
    corr = (rng.random(E) + 0.5).astype(F32)
    lt = torch.from_numpy(logits).to(dev)
    for mode, name in ((_lib.MASK_SINGLE, "single"), (_lib.MASK_MODULE, "module")):
        g = ops.gate_fused(logits=lt, top_k=k, expert_mask=torch.from_numpy(mask).to(dev), mask_mode=mode,
                           correction=torch.from_numpy(corr).to(dev), capacity=0, renorm_eps=1e-8)
        check_gate(g, logits, k, 0, E, expert_mask=mask, mask_mode=name, correction=corr, renorm_eps=1e-8)
        assert not np.isin(g.topk_idx.cpu().numpy(), [2, 5]).any()      # masked experts are never chosen
    bias = rng.standard_normal(E).astype(F32)
    g = ops.gate_fused(logits=lt, top_k=k, expert_mask=torch.from_numpy(bias).to(dev), mask_mode=_lib.MASK_BIAS,
                       temperature=0.7)
    check_gate(g, logits, k, 0, E, expert_mask=bias, mask_mode="bias", temperature=0.7)


def test_gate_ties_go_to_lowest_index(dev):
    from pikv_b200 import ops
    logits = np.zeros((64, 8), F32)
    logits[:, 5] = 1.0
    logits[10, :] = 0.0                      # fully tied row
    g = ops.gate_fused(logits=torch.from_numpy(logits).to(dev), top_k=3)
    gi = g.topk_idx.cpu().numpy()
    np.testing.assert_array_equal(gi[0], [5, 0, 1])
    np.testing.assert_array_equal(gi[10], [0, 1, 2])
    _, idx, _ = O.gate_tail(logits, 3)
    np.testing.assert_array_equal(gi, idx)


def test_gate_slot_base_and_capacity_drop(dev):
    from pikv_b200 import ops
    rng = np.random.default_rng(5)
    T, E, k, cap = 600, 4, 2, 200
    logits = rng.standard_normal((T, E)).astype(F32)
    base = np.array([0, 150, 199, 200], np.int32)
    g = ops.gate_fused(logits=torch.from_numpy(logits).to(dev), top_k=k, capacity=cap,
                       slot_base=torch.from_numpy(base).to(dev))
    gi = g.topk_idx.cpu().numpy()
    pos, counts_k = O.slot_assign_fast(gi, E, 1 << 30)
    want = pos + base[gi]
    want = np.where(want < cap, want, -1)
    np.testing.assert_array_equal(g.slot.cpu().numpy(), want)
    np.testing.assert_array_equal(g.new_len.cpu().numpy(), np.minimum(base + counts_k.sum(0), cap))
    assert (want[gi == 3] == -1).all()       # expert 3 was already full


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,E", [(256, 256, 4), (1000, 512, 8), (300, 1024, 64), (130, 72, 16)])
def test_gate_from_activations(dev, dtype, T, H, E):
    from pikv_b200 import ops
    torch.manual_seed(T + H)
    act = torch.relu(torch.randn(T, H)).to(dtype)
    w2 = (torch.randn(E, H) / H ** 0.5).to(dtype)
    b2 = torch.randn(E) * 0.1
    k = 2
    cap = O.capacity(T, 1.5, k, E)
    g = ops.gate_fused(act.to(dev), w2.to(dev), b2.to(dev), top_k=k, capacity=cap)
    logits = O.gate_logits(act.float().numpy(), w2.float().numpy(), b2.numpy())
    probs, idx, tw = O.gate_tail(logits, k)
    gi = g.topk_idx.cpu().numpy()
    same = (gi == idx).all(axis=1)
    margin = O.topk_margin(probs, k)
    # the GEMM's fp32 accumulation order differs from the CPU's: only near-ties may flip
    assert (same | (margin < 1e-4)).all()
    assert (~same).sum() <= max(1, T // 200)
    assert rel(g.probs.cpu().numpy(), probs) < 2e-5
    slot, counts_k = O.slot_assign_fast(gi, E, cap)
    np.testing.assert_array_equal(g.slot.cpu().numpy(), slot)
    np.testing.assert_array_equal(g.counts_k.cpu().numpy(), counts_k)


def test_gate_bf16_simt_and_tensor_core_paths_agree(dev):
    """bf16 activations normally take the tcgen05 kernel; the SIMT kernel must give the same experts
    and slots (near-ties aside) and probabilities within fp32 accumulation noise."""
    import pikv_b200
    from pikv_b200 import ops, _lib
    torch.manual_seed(21)
    T, H, E = 3000, 1024, 8
    act = torch.relu(torch.randn(T, H, device=dev)).bfloat16()
    w2 = (torch.randn(E, H, device=dev) / 32).bfloat16()
    tc = ops.gate_fused(act, w2, None, top_k=2, capacity=1200)
    torch.cuda.synchronize()
    assert pikv_b200.lib().pikv_gate_error_state() == 0
    simt = ops.gate_fused(act, w2, None, top_k=2, capacity=1200, phase=_lib.GATE_FORCE_SIMT)
    same = (tc.topk_idx == simt.topk_idx).all(dim=1)
    assert int((~same).sum()) <= 3
    assert torch.allclose(tc.probs, simt.probs, rtol=1e-4, atol=1e-7)
    if bool(same.all()):
        assert torch.equal(tc.slot, simt.slot) and torch.equal(tc.counts_k, simt.counts_k)


@pytest.mark.parametrize("T,H,E,k", [(128, 64, 8, 2), (129, 4096, 8, 2), (16384, 4096, 8, 2), (1000, 4096, 64, 2),
                                     (5000, 200, 20, 4), (200000, 128, 8, 2), (3000, 512, 40, 8), (2000, 256, 64, 8),
                                     (700, 320, 48, 3), (16384, 4096, 64, 2), (150000, 64, 64, 2), (4000, 128, 32, 1), (40000, 128, 24, 2)])
def test_gate_tensor_core_shapes(dev, T, H, E, k):
    """Ragged tiles, hidden sizes that are not multiples of 64, padded expert counts, several tiles per CTA."""
    import pikv_b200
    from pikv_b200 import ops
    torch.manual_seed(T)
    act = torch.relu(torch.randn(T, H, device=dev)).bfloat16()
    w2 = (torch.randn(E, H, device=dev) / H ** 0.5).bfloat16()
    b2 = torch.randn(E, device=dev) * 0.1
    cap = O.capacity(T, 1.25, k, E)
    g = ops.gate_fused(act, w2, b2, top_k=k, capacity=cap)
    torch.cuda.synchronize()
    assert pikv_b200.lib().pikv_gate_error_state() == 0
    logits = (act.float() @ w2.float().T + b2).cpu().numpy()
    probs, idx, tw = O.gate_tail(logits, k)
    gi = g.topk_idx.cpu().numpy()
    same = (gi == idx).all(axis=1)
    assert (same | (O.topk_margin(probs, k) < 1e-4)).all()
    assert rel(g.probs.cpu().numpy(), probs) < 2e-5
    slot, counts_k = O.slot_assign_fast(gi, E, cap)
    np.testing.assert_array_equal(g.slot.cpu().numpy(), slot)
    np.testing.assert_array_equal(g.counts_k.cpu().numpy(), counts_k)
    assert rel(g.prob_sum.cpu().numpy(), probs.sum(0)) < 1e-4


@pytest.mark.parametrize("E", [8, 24, 64])
def test_gate_tensor_core_ties_and_masks(dev, E):
    """Tied probabilities on the tensor-core path go to the lowest expert index, also when the tied experts sit in
    different 16-column groups of the shared-row tail; masks, correction and temperature follow the oracle."""
    import pikv_b200
    from pikv_b200 import ops, _lib
    T, H, k = 300, 128, 3
    act = torch.zeros(T, H, device=dev, dtype=torch.bfloat16)      # logits = bias exactly
    w2 = torch.ones(E, H, device=dev, dtype=torch.bfloat16)
    b2 = torch.zeros(E)
    b2[E - 1] = 1.0
    b2[3] = 1.0                                                     # experts 3 and E-1 tie for first, the rest for third
    g = ops.gate_fused(act, w2, b2.to(dev), top_k=k)
    torch.cuda.synchronize()
    assert pikv_b200.lib().pikv_gate_error_state() == 0
    gi = g.topk_idx.cpu().numpy()
    np.testing.assert_array_equal(gi, np.tile(np.array([3, E - 1, 0], dtype=np.int32), (T, 1)))
    logits = np.tile(b2.numpy(), (T, 1)).astype(np.float32)
    probs, idx, tw = O.gate_tail(logits, k)
    np.testing.assert_array_equal(gi, idx)
    assert rel(g.probs.cpu().numpy(), probs) < 1e-6
    assert rel(g.topk_w.cpu().numpy(), tw) < 1e-6
    # mask, correction, temperature against the oracle on random activations
    torch.manual_seed(E)
    act = torch.relu(torch.randn(T, H, device=dev)).bfloat16()
    w2 = (torch.randn(E, H, device=dev) / H ** 0.5).bfloat16()
    mask = (torch.rand(E) > 0.3).float()
    mask[:k] = 1.0
    corr = 0.5 + torch.rand(E)
    g = ops.gate_fused(act, w2, None, top_k=k, expert_mask=mask.to(dev), mask_mode=_lib.MASK_SINGLE,
                       correction=corr.to(dev), temperature=0.7, renorm_eps=1e-6)
    logits = (act.float() @ w2.float().T).cpu().numpy()
    probs, idx, tw = O.gate_tail(logits, k, expert_mask=mask.numpy(), mask_mode="single", correction=corr.numpy(),
                                 temperature=0.7, renorm_eps=1e-6)
    gi = g.topk_idx.cpu().numpy()
    same = (gi == idx).all(axis=1)
    assert (same | (O.topk_margin(probs, k) < 1e-4)).all()
    assert rel(g.probs.cpu().numpy(), probs) < 2e-5
    assert (mask.numpy()[gi] == 1.0).all()
    if same.all():
        assert rel(g.topk_w.cpu().numpy(), tw) < 2e-5


def test_gate_is_deterministic(dev):
    from pikv_b200 import ops
    torch.manual_seed(9)
    act = torch.randn(4096, 512, device=dev).bfloat16()
    w2 = torch.randn(8, 512, device=dev).bfloat16()
    a = ops.gate_fused(act, w2, None, top_k=2, capacity=1536)
    b = ops.gate_fused(act, w2, None, top_k=2, capacity=1536)
    for x, y in ((a.probs, b.probs), (a.slot, b.slot), (a.prob_sum, b.prob_sum), (a.topk_w, b.topk_w)):
        assert torch.equal(x, y)


# ---------------------------------------------------------------- router classes vs the reference's outputs
def load_sd(module, weights, dev):
    sd = {k: torch.from_numpy(np.array(v)) for k, v in weights.items()}
    module.load_state_dict(sd)
    return module.to(dev)


def test_base_router_matches_reference(dev):
    import pikv_b200
    g = load_golden("router_base_single")
    r = load_sd(pikv_b200.BaseRouter(64, 4, 2), sub(g, "weights"), dev)
    x = torch.from_numpy(g["x"]).to(dev)
    for tag, mask in (("", None), ("_m", torch.from_numpy(g["mask"]).to(dev))):
        d, c, p, aux = r(x, mask)
        assert rel(p.cpu().numpy(), g["probs" + tag]) < 1e-5
        np.testing.assert_array_equal(d.cpu().numpy(), g["dispatch" + tag])
        assert rel(c.cpu().numpy(), g["combine" + tag]) < 1e-5
        assert abs(float(aux) - float(g["aux" + tag])) < 1e-5 * max(1.0, abs(float(g["aux" + tag])))


@pytest.mark.parametrize("mode", ["entropy", "cv", "l2"])
def test_topk_balanced_router_matches_reference(dev, mode):
    import pikv_b200
    g = load_golden("router_topk_balanced_single")
    s = sub(g, mode)
    r = load_sd(pikv_b200.TopKBalancedRouter(64, 4, 2, balance_coefficient=0.01, balance_mode=mode), sub(s, "weights"), dev)
    d, c, p, aux = r(torch.from_numpy(g["x"]).to(dev))
    assert rel(p.cpu().numpy(), s["probs"]) < 1e-5
    np.testing.assert_array_equal(d.cpu().numpy(), s["dispatch"])
    assert rel(c.cpu().numpy(), s["combine"]) < 1e-5
    assert abs(float(aux) - float(s["aux"])) < 2e-5


def test_pikv_router_state_machine_matches_reference(dev):
    import pikv_b200
    g = load_golden("router_pikv_single")
    r = load_sd(pikv_b200.PiKVRouter(64, 4, 2, cache_update_interval=2), sub(g, "weights"), dev)
    kv = torch.from_numpy(g["kv"]).to(dev)
    with torch.no_grad():
        for i in range(3):
            c = sub(g, f"call{i}")
            d, cmb, p, aux, imp = r(torch.from_numpy(c["x"]).to(dev), kv_states=kv if i == 1 else None)
            assert rel(p.cpu().numpy(), c["probs"]) < 2e-5
            assert rel(imp.cpu().numpy(), c["importance"]) < 1e-5
            np.testing.assert_array_equal(d.cpu().numpy(), c["dispatch"])
            assert rel(cmb.cpu().numpy(), c["combine"]) < 2e-5
            assert rel(r.cache_usage_history.cpu().numpy(), c["history"]) < 1e-5
            assert rel(r.cache_correction_factor.detach().cpu().numpy(), c["factor"]) < 1e-5
            assert abs(float(aux) - float(c["aux"])) < 2e-5
    assert int(r.update_counter) == 3


def test_module_pikv_router_matches_reference(dev):
    """core/single/module PiKVRouter: cache-aware logit adjustment, predicted top-k, running-count slots."""
    from pikv_b200 import module as M
    g = load_golden("router_pikv_module")
    r = load_sd(M.PiKVRouter(32, 4, 2), sub(g, "weights"), dev)
    with torch.no_grad():
        d, c, p, aux, imp = r(torch.from_numpy(g["x"]).to(dev))
    assert rel(p.cpu().numpy(), g["probs"]) < 1e-5
    assert rel(imp.cpu().numpy(), g["importance"]) < 1e-5
    np.testing.assert_array_equal(d.cpu().numpy(), g["dispatch"])
    assert rel(c.cpu().numpy(), g["combine"]) < 1e-5
    assert abs(float(aux) - float(g["aux"])) < 1e-5
    np.testing.assert_array_equal(r.expert_usage_count.cpu().numpy(), g["usage"])


def test_module_adaptive_router_matches_reference(dev):
    """core/single/module AdaptiveRouter: importance-weighted combine tensor and the importance ring."""
    from pikv_b200 import module as M
    g = load_golden("router_adaptive_module")
    r = load_sd(M.AdaptiveRouter(32, 4, 2, importance_threshold=0.5), sub(g, "weights"), dev)
    with torch.no_grad():
        d, c, p, aux, imp = r(torch.from_numpy(g["x"]).to(dev))
    assert rel(p.cpu().numpy(), g["probs"]) < 1e-5
    assert rel(imp.cpu().numpy(), g["importance"]) < 1e-5
    np.testing.assert_array_equal(d.cpu().numpy(), g["dispatch"])
    assert rel(c.cpu().numpy(), g["combine"]) < 1e-5
    assert abs(float(aux) - float(g["aux"])) < 1e-5
    np.testing.assert_array_equal(r.expert_usage_count.cpu().numpy(), g["usage"])
    assert rel(r.importance_history.cpu().numpy(), g["history"]) < 1e-5
    assert int(r.importance_idx) == int(g["history_idx"])


def test_module_running_slots_match_reference_dispatch(dev):
    """The kernel's slot output reproduces the dense tensors core/single/module builds."""
    from pikv_b200 import ops
    g = load_golden("router_base_module")
    logits = g["logits"].reshape(-1, 4)
    cap = O.capacity(24, 1.0, 2, 4)
    res = ops.gate_fused(logits=torch.from_numpy(logits).to(dev), top_k=2, capacity=cap, renorm_eps=1e-8)
    d, c = ops.dispatch_scatter(res, 4, cap, position_mode=0)
    np.testing.assert_array_equal(d.cpu().numpy(), g["dispatch"].reshape(24, 4, cap))
    assert rel(c.cpu().numpy(), g["combine"].reshape(24, 4, cap)) < 1e-5
    np.testing.assert_array_equal(res.counts.cpu().numpy(), g["usage"].astype(np.int64))
    p_mean = res.prob_sum.cpu().numpy() / 24
    f = res.counts.cpu().numpy() / 48.0
    assert abs(float((p_mean * f).sum() * 4) - float(g["aux"])) < 1e-5


def test_gate_phases_on_two_streams(dev):
    """Scoring (phase 1) on one stream, slot finalisation (phase 2) on another after an event: the same
    result as the whole gate, for several batches in flight with their own workspaces."""
    from pikv_b200 import ops
    T, H, E, k = 5000, 512, 8, 2
    torch.manual_seed(3)
    w2 = (torch.randn(E, H, device=dev) / H ** 0.5).bfloat16()
    b2 = torch.randn(E, device=dev) * 0.1
    acts = [torch.relu(torch.randn(T, H, device=dev)).bfloat16() for _ in range(3)]
    base = torch.randint(0, 9, (E,), dtype=torch.int32, device=dev)
    want = [ops.gate_fused(a, w2, b2, top_k=k, capacity=1700, slot_base=base) for a in acts]
    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    got = []
    for a in acts:
        with torch.cuda.stream(s1):
            g = ops.gate_fused(a, w2, b2, top_k=k, capacity=1700, slot_base=base, phase=1)
            ev = torch.cuda.Event()
            ev.record(s1)
        s2.wait_event(ev)
        with torch.cuda.stream(s2):
            ops.gate_fused(a, w2, b2, top_k=k, capacity=1700, slot_base=base, phase=2, out=g)
        got.append(g)
    torch.cuda.synchronize()
    for w, g in zip(want, got):
        for name in ("probs", "topk_idx", "topk_w", "slot", "counts_k", "prob_sum", "new_len"):
            assert torch.equal(getattr(w, name), getattr(g, name)), name


@pytest.mark.parametrize("T,K,H,E,k", [(128, 64, 256, 8, 2), (1000, 512, 768, 8, 2), (4096, 4096, 4096, 8, 2),
                                       (300, 256, 296, 20, 4), (2048, 1024, 1024, 32, 2)])
def test_gate_mlp_fused_matches_oracle(dev, T, K, H, E, k):
    """Both layers of the gate net and the tail in one tensor-core kernel (pikv_gate_mlp_fused) against the oracle:
    hidden = bf16(relu(x w1^T + b1)), logits = hidden w2^T + b2 in fp32, then the gate tail.  Expert indices equal
    except at near-ties of the oracle's top-k (counted), probabilities within 1e-2, slots exact on the GPU's indices."""
    import pikv_b200
    from pikv_b200 import ops
    g0 = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, K, generator=g0).bfloat16()
    w1 = ((torch.rand(H, K, generator=g0) * 2 - 1) / K ** 0.5).bfloat16()
    b1 = (torch.rand(H, generator=g0) * 2 - 1) / K ** 0.5
    w2 = ((torch.rand(E, H, generator=g0) * 2 - 1) / H ** 0.5 * 4).bfloat16()
    b2 = (torch.rand(E, generator=g0) * 2 - 1) / H ** 0.5
    cap = max(4, int(T * 1.5 * k / E))
    res = ops.gate_mlp_fused(x.to(dev), w1.to(dev), b1.to(dev), w2.to(dev), b2.to(dev), top_k=k, capacity=cap)
    torch.cuda.synchronize()
    assert pikv_b200.lib().pikv_gate_error_state() == 0
    hid = np.maximum(x.float().numpy() @ w1.float().numpy().T + b1.numpy(), 0).astype(np.float32)
    logits = O.gate_logits(O.bf16_round(hid), w2.float().numpy(), b2.numpy())
    probs, idx, tw = O.gate_tail(logits, k)
    gi = res.topk_idx.cpu().numpy()
    diff = (gi != idx).any(axis=1)
    # the hidden activations are rounded to bf16 after an fp32 sum in another order: a rounding flip moves a logit by
    # up to ~1e-3, so "near-tie" is judged on that scale, between any two neighbours of the sorted top k+1 (a flip
    # of the first two choices is a mismatch of the ordered index pair too)
    srt = -np.sort(-probs, axis=1)[:, : k + 1]
    gap = ((srt[:, :-1] - srt[:, 1:]) / np.maximum(srt[:, :-1], 1e-30)).min(axis=1)
    assert (gap[diff] < 2e-2).all() and diff.sum() <= max(2, T // 50), int(diff.sum())
    assert np.abs(res.probs.cpu().numpy() - probs).max() < 1e-2
    slot, counts_k = O.slot_assign_fast(gi, E, cap)
    np.testing.assert_array_equal(res.slot.cpu().numpy(), slot)
    np.testing.assert_array_equal(res.counts_k.cpu().numpy(), counts_k)
    np.testing.assert_array_equal(res.new_len.cpu().numpy(), np.minimum(counts_k.sum(0), cap))
    assert abs(float(res.prob_sum.sum()) - T) < 1e-2 * T
    again = ops.gate_mlp_fused(x.to(dev), w1.to(dev), b1.to(dev), w2.to(dev), b2.to(dev), top_k=k, capacity=cap)
    assert torch.equal(again.probs, res.probs) and torch.equal(again.slot, res.slot)      # run-to-run identical bits


def test_base_router_bf16_uses_fused_gate_net(dev):
    """A bf16 BaseRouter runs its gate net in the fused kernel; its experts agree with the fp32 path of the same
    weights except at near-ties."""
    import pikv_b200
    torch.manual_seed(3)
    r32 = pikv_b200.BaseRouter(256, 8, top_k=2).to(dev).eval()
    r16 = pikv_b200.BaseRouter(256, 8, top_k=2).to(dev).eval()
    r16.load_state_dict(r32.state_dict())
    x = torch.randn(4, 64, 256, device=dev)
    with torch.no_grad():
        before = pikv_b200.launch_count()
        r16(x.bfloat16())
        assert pikv_b200.launch_count() - before >= 2
        r32(x)
    a, b = r16.last_gate.topk_idx, r32.last_gate.topk_idx
    assert float((a != b).any(dim=1).float().mean()) < 0.05
    assert torch.allclose(r16.last_gate.probs, r32.last_gate.probs, atol=2e-2)
