"""GPU parity: quantised routed append, block-wide fake quantisation, H2O select / compact,
decode attention, record pack / unpack - against the oracle and the reference's golden vectors."""
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


def outlier_kv(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g)
    cols = torch.randperm(H, generator=g)[: max(1, round(0.01 * H))]
    x[:, cols] *= 20.0
    return x.bfloat16()


def read_all(cache, lens, which):
    E, cap = cache.num_seqs, cache.capacity
    seq = np.repeat(np.arange(E), cap).astype(np.int32)
    pos = np.tile(np.arange(cap), E).astype(np.int32)
    valid = pos < lens[seq]
    dev = cache.k_codes.device
    dq, codes = cache.gather(torch.from_numpy(seq[valid]).to(dev), torch.from_numpy(pos[valid]).to(dev), which, codes=True)
    return seq[valid], pos[valid], dq.cpu().numpy(), codes.cpu().numpy()


# ---------------------------------------------------------------- append
@pytest.mark.parametrize("bits,sym", [(8, True), (4, False), (8, False), (4, True)])
@pytest.mark.parametrize("T,E,k,n_kv", [(300, 4, 2, 2), (2048, 8, 2, 8), (17, 3, 1, 1)])
def test_append_codes_bit_exact(dev, bits, sym, T, E, k, n_kv):
    import pikv_b200
    H = n_kv * 128
    K, V = outlier_kv(T, H, 1), outlier_kv(T, H, 2)
    rng = np.random.default_rng(T)
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    cap = max(16, int(T * 1.2 * k / E))                       # tight: some pairs are dropped
    slot, counts_k = O.slot_assign_fast(idx, E, cap)
    cache = pikv_b200.PagedKVCache(E, cap, n_kv, bits=bits, symmetric=sym, device=dev)
    cache.append(K.to(dev), V.to(dev), torch.from_numpy(idx).to(dev), torch.from_numpy(slot).to(dev))
    torch.cuda.synchronize()
    cache.check_status()
    ref = O.routed_append(K.float().numpy(), V.float().numpy(), idx, slot, E, cap, bits, sym, 128)
    lens = ref["length"]
    for which in ("k", "v"):
        s, p, dq, codes = read_all(cache, lens, which)
        if not sym:
            codes = codes.view(np.uint8)        # asymmetric codes are unsigned bytes
        np.testing.assert_array_equal(codes.astype(F32), ref[f"{which}_codes"][s, p])
        # stored scale = bf16(fp32 scale); stored zero point exact
        sc = O.bf16_round(ref[f"{which}_scale"][s, p])
        want = O.dequant_token_groups(ref[f"{which}_codes"][s, p], sc, ref[f"{which}_zp"][s, p], 128)
        np.testing.assert_array_equal(dq, want)
        # and the bf16 scale costs < 2^-8 relative against the reference's own dequantised values
        full = O.dequant_token_groups(ref[f"{which}_codes"][s, p], ref[f"{which}_scale"][s, p], ref[f"{which}_zp"][s, p], 128)
        assert np.abs(dq - full).max() <= np.abs(full).max() * 2.0 ** -8


def test_append_matches_reference_slices(dev):
    """Codes of the reference's own _quantize_tensor on [1,128] slices (golden), including an all-zero
    slice, a constant slice and a slice with a large offset."""
    import pikv_b200
    g = load_golden("quant_slices")
    x = torch.from_numpy(g["x"]).bfloat16()
    T = x.shape[0]
    idx = torch.zeros(T, 1, dtype=torch.int32)
    slot = torch.arange(T, dtype=torch.int32)[:, None]
    for tag, bits, sym in (("int8_sym", 8, True), ("int4_asym", 4, False), ("int8_asym", 8, False), ("int4_sym", 4, True)):
        cache = pikv_b200.PagedKVCache(1, 16, 2, bits=bits, symmetric=sym, device=dev)
        cache.append(x.to(dev), x.to(dev), idx.to(dev), slot.to(dev))
        _, codes = cache.gather(idx[:, 0].to(dev), slot[:, 0].to(dev), "k", codes=True)
        codes = codes.cpu().numpy()
        if not sym:
            codes = codes.view(np.uint8)
        np.testing.assert_array_equal(codes.astype(F32), g[f"{tag}/q"])
        np.testing.assert_array_equal(cache.k_codes.cpu().numpy(), cache.v_codes.cpu().numpy())
        cache.check_status()


def test_append_fp32_input_and_empty(dev):
    import pikv_b200
    cache = pikv_b200.PagedKVCache(2, 32, 1, device=dev)
    x = torch.randn(20, 128)
    idx = torch.zeros(20, 1, dtype=torch.int32)
    slot = torch.arange(20, dtype=torch.int32)[:, None]
    cache.append(x.to(dev), x.to(dev), idx.to(dev), slot.to(dev))
    q, sc, zp = O.quant_token_groups(x.numpy(), 8, 128, True)
    _, codes = cache.gather(idx[:, 0].to(dev), slot[:, 0].to(dev), "k", codes=True)
    np.testing.assert_array_equal(codes.cpu().numpy().astype(F32), q)
    cache.append(x[:0].to(dev), x[:0].to(dev), idx[:0].to(dev), slot[:0].to(dev))     # empty batch is a no-op
    cache.check_status()


def test_append_flags_bad_destination(dev):
    import pikv_b200
    cache = pikv_b200.PagedKVCache(2, 32, 1, device=dev)
    x = torch.randn(4, 128, device=dev).bfloat16()
    idx = torch.tensor([[0], [7], [1], [0]], dtype=torch.int32, device=dev)       # 7 is not a sequence
    slot = torch.tensor([[0], [0], [0], [1]], dtype=torch.int32, device=dev)
    cache.append(x, x, idx, slot)
    with pytest.raises(pikv_b200.PikvError):
        cache.check_status()


def test_full_size_append_matches_oracle(dev):
    """Config 2 at full size (16384 tokens, hidden 4096, 8 experts top-2, 8 KV heads) against the oracle: expert
    indices equal except at near-ties of the oracle's top-k (counted); on the GPU's own indices the slots,
    counts and lengths are equal and every stored code and scale is bit-exact, for int8 symmetric and 4-bit
    asymmetric caches."""
    import pikv_b200
    from pikv_b200 import ops
    T, H, E, k, n_kv = 16384, 4096, 8, 2, 8
    g0 = torch.Generator().manual_seed(0)
    act = torch.randn(T, H, generator=g0).bfloat16()
    w2 = (torch.randn(E, H, generator=g0) / 64).bfloat16()
    K, V = outlier_kv(T, n_kv * 128, 3), outlier_kv(T, n_kv * 128, 4)
    cap = O.capacity(T, 1.5, k, E)
    g = ops.gate_fused(act.to(dev), w2.to(dev), None, top_k=k, capacity=cap)
    logits = O.gate_logits(act.float().numpy(), w2.float().numpy(), None)
    probs, idx, _ = O.gate_tail(logits, k)
    gi = g.topk_idx.cpu().numpy()
    diff = (gi != idx).any(axis=1)
    assert (O.topk_margin(probs, k)[diff] < 1e-4).all() and diff.sum() <= T // 200, f"{int(diff.sum())} index mismatches"
    print(f"config 2: {int(diff.sum())} of {T} tokens differ from the oracle's experts, all near-ties")
    slot, counts_k = O.slot_assign_fast(gi, E, cap)
    np.testing.assert_array_equal(g.slot.cpu().numpy(), slot)
    np.testing.assert_array_equal(g.counts_k.cpu().numpy(), counts_k)
    Kf, Vf = K.float().numpy(), V.float().numpy()
    for bits, sym in ((8, True), (4, False)):
        cache = pikv_b200.PagedKVCache(E, cap, n_kv, bits=bits, symmetric=sym, device=dev)
        cache.append(K.to(dev), V.to(dev), g.topk_idx, g.slot)
        cache.length.copy_(g.new_len)
        cache.check_status()
        ref = O.routed_append(Kf, Vf, gi, slot, E, cap, bits, sym, 128)
        lens = ref["length"]
        np.testing.assert_array_equal(g.new_len.cpu().numpy(), lens)
        for which, name in (("k", "k"), ("v", "v")):
            sq, ps, dq, codes = read_all(cache, lens, which)
            np.testing.assert_array_equal(codes.astype(F32), ref[f"{name}_codes"][sq, ps])
            sc = O.bf16_round(ref[f"{name}_scale"][sq, ps])
            want = O.dequant_token_groups(ref[f"{name}_codes"][sq, ps], sc, ref[f"{name}_zp"][sq, ps], 128)
            np.testing.assert_array_equal(dq, want)             # (code - zp) * stored scale: scales and zero points too
        del cache


def test_full_size_decode_matches_oracle(dev):
    """Config 3 at full size: 64 streams x 32 query / 8 KV heads x context 32768 in one call with the
    library's default split count; three streams (first, middle, last: the page-table stride and the 4.3 GB
    offsets) are compared with the oracle on the dequantised cache at 1e-2, int8 and 4-bit caches."""
    import pikv_b200
    B, n_q, n_kv, ctx = 64, 32, 8, 32768
    for bits in (8, 4):
        cache = pikv_b200.PagedKVCache(B, ctx, n_kv, bits=bits, symmetric=(bits == 8), device=dev)
        gen = torch.Generator(device=dev).manual_seed(11)
        pos = torch.arange(ctx, dtype=torch.int32, device=dev)[:, None].contiguous()
        for b in range(B):
            K = torch.randn(ctx, n_kv * 128, generator=gen, device=dev).bfloat16()
            V = torch.randn(ctx, n_kv * 128, generator=gen, device=dev).bfloat16()
            cache.append(K, V, torch.full((ctx, 1), b, dtype=torch.int32, device=dev), pos)
        lens = torch.full((B,), ctx, dtype=torch.int32)
        lens[31] = ctx - 4321                                   # one ragged stream among the full ones
        cache.length.copy_(lens.to(dev))
        q = torch.randn(B, n_q, 128, generator=gen, device=dev).bfloat16()
        out = cache.decode_attention(q)
        torch.cuda.synchronize()
        cache.check_status()
        got = out.float().cpu().numpy()
        for b in (0, 31, 63):
            n = int(lens[b])
            seq = torch.full((n,), b, dtype=torch.int32, device=dev)
            kd = cache.gather(seq, pos[:n, 0].contiguous(), "k").cpu().numpy().reshape(1, n, n_kv, 128).transpose(0, 2, 1, 3)
            vd = cache.gather(seq, pos[:n, 0].contiguous(), "v").cpu().numpy().reshape(1, n, n_kv, 128).transpose(0, 2, 1, 3)
            want, _ = O.decode_attention(q[b:b + 1].float().cpu().numpy(), kd, vd, np.array([n]))
            assert np.abs(got[b] - want[0]).max() <= 1e-2 * np.abs(want).max(), (bits, b)
        del cache
        torch.cuda.empty_cache()


# ---------------------------------------------------------------- block-wide fake quantisation
@pytest.mark.parametrize("tag,bits,gs,sym,single", [
    ("single_b8g1", 8, 1, False, True), ("single_b4g16", 4, 16, False, True), ("single_b8g64", 8, 64, False, True),
    ("module_b8g32s", 8, 32, True, False), ("module_b4g32a", 4, 32, False, False),
    ("module_b4g16s", 4, 16, True, False), ("module_b8g64a", 8, 64, False, False)])
def test_quant_block_matches_reference(dev, tag, bits, gs, sym, single):
    import pikv_b200
    from pikv_b200.module import compression as mc
    g = load_golden("quant_block")
    k, v = torch.from_numpy(g["keys"]).to(dev), torch.from_numpy(g["values"]).to(dev)
    qc = (pikv_b200.QuantizedCompressor(64, bits=bits, group_size=gs) if single
          else mc.QuantizedCompressor(64, bits=bits, group_size=gs, symmetric=sym)).to(dev)
    dk, dv = qc(k, v)
    np.testing.assert_array_equal(dk.cpu().numpy(), g[f"{tag}/dq_keys"])
    np.testing.assert_array_equal(dv.cpu().numpy(), g[f"{tag}/dq_values"])
    assert rel(float(qc.quantization_error), float(g[f"{tag}/quantization_error"])) < 1e-5
    if single:
        assert float(qc.sample_count) == float(g[f"{tag}/sample_count"])


def test_quant_block_static_mode_matches_reference(dev):
    import pikv_b200
    g = load_golden("quant_block")
    qc = pikv_b200.QuantizedCompressor(64, bits=8, group_size=16, dynamic_quantization=False).to(dev)
    dk, dv = qc(torch.from_numpy(g["keys"]).to(dev), torch.from_numpy(g["values"]).to(dev))
    np.testing.assert_array_equal(dk.cpu().numpy(), g["single_static/dq_keys"])
    np.testing.assert_array_equal(dv.cpu().numpy(), g["single_static/dq_values"])
    assert float(qc.scale) == float(g["single_static/scale"])


def test_quant_block_large_bf16(dev):
    from pikv_b200 import ops
    x = outlier_kv(4099, 1024, 7)
    dq, q, params, err = ops.quant_block(x.to(dev), 128, -128, 127, True, want_codes=True)
    rdq, rq, rs, rz, _ = O.quant_block_forward(x.float().numpy(), 8, 128, True)
    np.testing.assert_array_equal(q.cpu().numpy(), rq)
    np.testing.assert_array_equal(dq.cpu().numpy(), rdq)
    np.testing.assert_array_equal(params[:, 0].cpu().numpy(), rs)


# ---------------------------------------------------------------- H2O
def test_h2o_select_matches_reference_and_oracle(dev):
    import pikv_b200
    from pikv_b200 import ops
    g = load_golden("h2o_select")
    n = int(g["n"])
    sch = pikv_b200.H2OScheduler(256, 16, heavy_ratio=0.1, recent_ratio=0.05).to(dev)
    sch.attention_accumulator.copy_(torch.from_numpy(g["acc"]))
    sch.access_timestamps.copy_(torch.from_numpy(g["ts"]))
    keys = torch.zeros(n, 16, device=dev)
    mask = sch.select_eviction_candidates(keys, keys, {})
    np.testing.assert_array_equal(mask.cpu().numpy(), g["evict_mask"])
    kept = int(sch.last_kept_count.item())
    np.testing.assert_array_equal(sch.last_keep_idx[:kept].cpu().numpy(), np.nonzero(~g["evict_mask"])[0])


@pytest.mark.parametrize("n,nh,nr,levels", [(1000, 100, 50, 0), (32768, 1792, 256, 0), (32768, 1792, 256, 8),
                                            (5000, 1, 1, 3), (777, 777, 5, 0), (60000, 3000, 100, 16)])
def test_h2o_select_segments_and_ties(dev, n, nh, nr, levels):
    from pikv_b200 import ops
    rng = np.random.default_rng(n + levels)
    S = 5
    acc = rng.random((S, n)).astype(F32) - 0.25
    if levels:
        acc = np.floor(acc * levels).astype(F32) / levels           # heavy ties
    ts = np.tile(np.arange(n, dtype=F32), (S, 1))
    ts[1] = rng.permutation(n).astype(F32)
    ts[2] = np.floor(ts[2] / 7)                                      # tied timestamps
    mask, keep, cnt = ops.h2o_select(torch.from_numpy(acc).to(dev), torch.from_numpy(ts).to(dev), nh, nr)
    for s in range(S):
        ev, ki = O.h2o_select(acc[s], ts[s], nh, nr)
        np.testing.assert_array_equal(mask[s].cpu().numpy(), ev)
        assert int(cnt[s]) == len(ki)
        np.testing.assert_array_equal(keep[s, : len(ki)].cpu().numpy(), ki)


@pytest.mark.parametrize("kind", ["uniform", "heavy_tail", "outlier", "levels", "ascending", "ascending_runs", "constant",
                                  "dense_bucket", "unaligned", "signed_zeros"])
def test_h2o_select_routines_agree_with_oracle(dev, kind):
    """The streaming select (the default), the two radix routines and the bucketed select on staged keys must all
    return the oracle's mask on score distributions that stress them differently: a far outlier (every other key
    in one bucket), eight tied levels, keys already in ascending order (range marks), runs of equal timestamps."""
    import pikv_b200
    from pikv_b200 import ops
    rng = np.random.default_rng(5)
    S, n, nh, nr = 5, 5000, 300, 40
    acc = {"uniform": rng.random((S, n)), "heavy_tail": rng.pareto(1.2, (S, n)), "outlier": rng.random((S, n)),
           "levels": rng.integers(0, 8, (S, n)) / 8.0, "ascending": np.sort(rng.random((S, n)), axis=1),
           "ascending_runs": np.sort(rng.integers(0, 50, (S, n)), axis=1).astype(np.float64),
           "constant": np.full((S, n), 0.25),
           # thousands of distinct keys inside one first-level bucket beside a wide spread: narrowed pass by pass
           "dense_bucket": np.where(rng.random((S, n)) < 0.04, rng.random((S, n)) * 1e6, 1.0 + rng.random((S, n)) * 1e-4),
           "unaligned": rng.random((S, n)),
           # -0.0 and +0.0 are one value: the cut falls inside them and the lowest indices must win
           "signed_zeros": np.where(rng.random((S, n)) < 0.03, 0.5 + rng.random((S, n)), 0.0)}[kind].astype(F32)
    if kind == "signed_zeros":
        neg = rng.random((S, n)) < 0.5
        acc = np.where((acc == 0) & neg, np.float32(-0.0), acc).astype(F32)
    if kind == "unaligned":
        n = 4999                                               # rows that start off a 16-byte boundary
        acc = np.ascontiguousarray(acc[:, :n])
    if kind == "outlier":
        acc[:, 7] = 1e30
        acc[:, 11] = -1e30
    ts = np.tile(np.arange(n, dtype=F32), (S, 1))
    if kind == "ascending_runs":
        ts = np.floor(ts / 16)                                 # timestamps in runs of 16 equal values
    if kind == "levels":
        ts = rng.permutation(n).astype(F32)[None].repeat(S, 0)
    want = np.stack([O.h2o_select(acc[s], ts[s], nh, nr)[0] for s in range(S)])
    a, t = torch.from_numpy(acc).to(dev), torch.from_numpy(ts).to(dev)
    try:
        for variant in (0, 1, 2, 3):
            assert pikv_b200.lib().pikv_h2o_select_variant(variant) == 0
            mask, keep, cnt = ops.h2o_select(a, t, nh, nr)
            np.testing.assert_array_equal(mask.cpu().numpy(), want, err_msg=f"variant {variant}")
            for s in range(S):
                kept = np.nonzero(~want[s])[0]
                assert int(cnt[s]) == len(kept)
                np.testing.assert_array_equal(keep[s, : len(kept)].cpu().numpy(), kept)
    finally:
        pikv_b200.lib().pikv_h2o_select_variant(0)


def test_h2o_select_ragged_lengths(dev):
    from pikv_b200 import ops
    rng = np.random.default_rng(1)
    lens = np.array([0, 1, 16, 100, 512], np.int32)
    acc = rng.random((5, 512)).astype(F32)
    ts = np.tile(np.arange(512, dtype=F32), (5, 1))
    mask, keep, cnt = ops.h2o_select(torch.from_numpy(acc).to(dev), torch.from_numpy(ts).to(dev), 20, 10,
                                     seg_len=torch.from_numpy(lens).to(dev))
    for s, n in enumerate(lens):
        ev = np.ones(512, bool)
        if n:
            ev[:n], ki = O.h2o_select(acc[s, :n], ts[s, :n], 20, 10)
        else:
            ki = np.zeros(0, np.int32)
        np.testing.assert_array_equal(mask[s].cpu().numpy(), ev)
        np.testing.assert_array_equal(keep[s, : len(ki)].cpu().numpy(), ki)
        assert int(cnt[s]) == len(ki)


def test_h2o_accumulate(dev):
    import pikv_b200
    sch = pikv_b200.H2OScheduler(128, 8).to(dev)
    acc, ts, t = np.zeros(128, F32), np.zeros(128, F32), 0
    rng = np.random.default_rng(2)
    for _ in range(4):
        ix = rng.permutation(128)[:40]
        w = rng.random(40).astype(F32)
        sch.update_attention_scores(torch.from_numpy(ix).to(dev), torch.from_numpy(w).to(dev))
        t = O.h2o_update(acc, ts, t, ix, w)
    np.testing.assert_array_equal(sch.attention_accumulator.cpu().numpy(), acc)
    np.testing.assert_array_equal(sch.access_timestamps.cpu().numpy(), ts)
    assert int(sch.current_time) == 4


def test_manager_sequence_matches_reference(dev):
    import pikv_b200
    g = load_golden("h2o_manager")
    mgr = pikv_b200.CacheSchedulingManager(64, 8, pikv_b200.SchedulingPolicy.H2O).to(dev)
    for s in range(5):
        c = sub(g, f"s{s}")
        mgr.scheduler.attention_accumulator.copy_(torch.from_numpy(c["acc"]))
        mgr.scheduler.access_timestamps.copy_(torch.from_numpy(c["ts"]))
        mgr.update_cache(torch.from_numpy(c["keys_in"]).to(dev), torch.from_numpy(c["values_in"]).to(dev))
        size = int(c["size"])
        assert int(mgr.cache_size_current) == size
        np.testing.assert_array_equal(mgr.cache_keys[:size].cpu().numpy(), c["cache_keys"][:size])
        np.testing.assert_array_equal(mgr.cache_values[:size].cpu().numpy(), c["cache_values"][:size])
        assert int(mgr.scheduler.eviction_count) == int(c["evictions"])


# ---------------------------------------------------------------- decode attention
def fill_stream_cache(dev, B, n_kv, ctx, lens, seed, bits=8, symmetric=True, shift=0.0):
    import pikv_b200
    torch.manual_seed(seed)
    cache = pikv_b200.PagedKVCache(B, ctx, n_kv, bits=bits, symmetric=symmetric, device=dev)
    # shuffle the physical pages so the page table is really used
    perm = torch.randperm(cache.num_pages, device=dev).to(torch.int32)
    cache.page_table.copy_(perm.view(B, -1))
    K = (torch.randn(B * ctx, n_kv * 128) + shift).bfloat16()
    V = (torch.randn(B * ctx, n_kv * 128) * (1.0 + shift) - shift).bfloat16()
    if shift:
        K[min(5, B * ctx - 1)] = 3.0      # constant rows: the reference's zero point runs into the millions
        V[min(7, B * ctx - 1)] = -2.0
    seq = torch.arange(B, dtype=torch.int32).repeat_interleave(ctx)[:, None]
    pos = torch.arange(ctx, dtype=torch.int32).repeat(B)[:, None]
    cache.append(K.to(dev), V.to(dev), seq.to(dev), pos.to(dev))
    cache.length.copy_(torch.from_numpy(lens).to(dev))
    kd = cache.gather(seq[:, 0].to(dev), pos[:, 0].to(dev), "k").cpu().numpy().reshape(B, ctx, n_kv, 128).transpose(0, 2, 1, 3)
    vd = cache.gather(seq[:, 0].to(dev), pos[:, 0].to(dev), "v").cpu().numpy().reshape(B, ctx, n_kv, 128).transpose(0, 2, 1, 3)
    return cache, kd, vd


@pytest.mark.parametrize("B,n_q,n_kv,ctx,splits", [(2, 8, 2, 100, 1), (3, 8, 2, 1000, 3), (2, 4, 4, 257, 2),
                                                    (2, 16, 2, 640, 0), (1, 32, 8, 4096, 4), (4, 2, 2, 48, 5)])
def test_decode_attention_matches_oracle(dev, B, n_q, n_kv, ctx, splits):
    rng = np.random.default_rng(ctx)
    lens = rng.integers(1, ctx + 1, B).astype(np.int32)
    lens[0] = ctx
    cache, kd, vd = fill_stream_cache(dev, B, n_kv, ctx, lens, ctx)
    q = torch.randn(B, n_q, 128).bfloat16()
    out, lse = cache.decode_attention(q.to(dev), splits=splits, want_lse=True)
    cache.check_status()
    want, _ = O.decode_attention(q.float().numpy(), kd, vd, lens)
    got = out.float().cpu().numpy()
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    # log-sum-exp of the scaled scores
    for b in range(B):
        g = n_q // n_kv
        for h in range(n_q):
            s = (q[b, h].float().numpy() @ kd[b, h // g, : lens[b]].T) / np.sqrt(128.0)
            ref = np.log(np.exp(s - s.max()).sum()) + s.max()
            assert abs(float(lse[b, h]) - ref) < 1e-3 * max(1.0, abs(ref))


@pytest.mark.parametrize("B,n_q,n_kv,ctx,splits", [(2, 8, 2, 100, 1), (3, 8, 2, 1000, 3), (2, 4, 4, 257, 2),
                                                    (2, 16, 2, 640, 0), (1, 32, 8, 4096, 4), (4, 2, 2, 48, 5)])
def test_decode_attention_q4_matches_oracle(dev, B, n_q, n_kv, ctx, splits):
    """4-bit asymmetric cache: the oracle attends over the dequantised (code - zp) * scale rows, so only the
    kernel's arithmetic (f16 operands, zero point carried beside the tensor-core sums) is under test."""
    rng = np.random.default_rng(ctx + 1)
    lens = rng.integers(1, ctx + 1, B).astype(np.int32)
    lens[0] = ctx
    cache, kd, vd = fill_stream_cache(dev, B, n_kv, ctx, lens, ctx, bits=4, symmetric=False, shift=0.75)
    q = torch.randn(B, n_q, 128).bfloat16()
    out, lse = cache.decode_attention(q.to(dev), splits=splits, want_lse=True)
    cache.check_status()
    want, _ = O.decode_attention(q.float().numpy(), kd, vd, lens)
    got = out.float().cpu().numpy()
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    g = n_q // n_kv
    for b in range(B):
        for h in range(n_q):
            sc = (q[b, h].float().numpy() @ kd[b, h // g, : lens[b]].T) / np.sqrt(128.0)
            ref = np.log(np.exp(sc - sc.max()).sum()) + sc.max()
            assert abs(float(lse[b, h]) - ref) < 1e-3 * max(1.0, abs(ref))


def test_decode_attention_reference_mha_fixture(dev):
    """1:1 heads, the reference's own _compute_attention output; the cache adds only int8 error."""
    g = load_golden("attention_decode")
    import pikv_b200
    q = torch.from_numpy(g["q"][:, 0])
    B, heads, d = q.shape
    # the fixture has 16-wide heads; embed them in the first 16 of 128 channels (zeros elsewhere do not
    # change q.k, and the 1/sqrt(d) factor is re-scaled through q)
    ctx = g["k"].shape[1]
    K = torch.zeros(B * ctx, heads * 128)
    V = torch.zeros(B * ctx, heads * 128)
    kk = torch.from_numpy(g["k"]).reshape(B * ctx, heads, 16)
    vv = torch.from_numpy(g["v"]).reshape(B * ctx, heads, 16)
    K.view(-1, heads, 128)[:, :, :16] = kk
    V.view(-1, heads, 128)[:, :, :16] = vv
    qq = torch.zeros(B, heads, 128)
    qq[:, :, :16] = q * (128.0 / 16.0) ** 0.5
    cache = pikv_b200.PagedKVCache(B, ctx, heads, device=dev)
    seq = torch.arange(B, dtype=torch.int32).repeat_interleave(ctx)[:, None].to(dev)
    pos = torch.arange(ctx, dtype=torch.int32).repeat(B)[:, None].to(dev)
    cache.append(K.to(dev), V.to(dev), seq, pos)
    cache.length.fill_(ctx)
    out = cache.decode_attention(qq.bfloat16().to(dev)).float().cpu().numpy()[:, :, :16]
    want = g["context"][:, 0]
    assert np.abs(out - want).max() <= 3e-2 * np.abs(want).max()     # int8 cache + bf16 q/out vs the fp32 reference


def test_decode_scores_feed_h2o_accumulate(dev):
    from pikv_b200 import ops
    B, n_q, n_kv, ctx = 2, 8, 2, 300
    lens = np.array([300, 123], np.int32)
    cache, kd, vd = fill_stream_cache(dev, B, n_kv, ctx, lens, 11)
    q = torch.randn(B, n_q, 128).bfloat16()
    scores = torch.zeros(B, n_q, ctx, device=dev)
    out, lse = cache.decode_attention(q.to(dev), splits=2, scores=scores)
    acc = torch.zeros(B * n_kv, ctx, device=dev)
    ops.h2o_accumulate_attn(scores, lse, cache.length, n_kv, acc)
    _, psum = O.decode_attention(q.float().numpy(), kd, vd, lens)
    got = acc.cpu().numpy().reshape(B, n_kv, ctx)
    assert np.abs(got - psum).max() < 1e-4
    assert np.abs(got.sum(-1) - n_q // n_kv).max() < 1e-3           # probabilities of each query head sum to 1


@pytest.mark.parametrize("B,n_q,n_kv,ctx", [(2, 8, 2, 300), (3, 16, 2, 1000), (2, 4, 4, 77)])
def test_decode_h2o_update_from_compact_probabilities(dev, B, n_q, n_kv, ctx):
    """The fused H2O update: the decode kernel's f16 probabilities (relative to their softmax step) normalised by
    pikv_h2o_accumulate_probs equal the oracle's column sums of the attention probabilities within 1e-2 relative
    (f16 carries 11 bits), and each query head's probabilities still sum to one."""
    rng = np.random.default_rng(ctx)
    lens = rng.integers(1, ctx + 1, B).astype(np.int32)
    lens[0] = ctx
    cache, kd, vd = fill_stream_cache(dev, B, n_kv, ctx, lens, ctx + 1)
    q = torch.randn(B, n_q, 128).bfloat16()
    acc = torch.zeros(B * n_kv, ctx, device=dev)
    out = cache.decode_attention_h2o(q.to(dev), acc)
    want_out, psum = O.decode_attention(q.float().numpy(), kd, vd, lens)
    got = acc.cpu().numpy().reshape(B, n_kv, ctx)
    assert np.abs(got - psum).max() <= 1e-2 * max(psum.max(), 1e-6)
    assert np.abs(got.sum(-1) - n_q // n_kv).max() < 2e-3
    assert np.abs(out.float().cpu().numpy() - want_out).max() <= 1e-2 * np.abs(want_out).max()
    cache.decode_attention_h2o(q.to(dev), acc)                  # accumulates
    assert np.abs(acc.cpu().numpy().reshape(B, n_kv, ctx) - 2 * psum).max() <= 2e-2 * max(psum.max(), 1e-6)


# ---------------------------------------------------------------- compaction
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("per_head", [True, False])
def test_h2o_compact_moves_rows_and_scores(dev, per_head, bits):
    import pikv_b200
    from pikv_b200 import ops
    B, n_kv, ctx = 3, 2, 200
    lens = np.array([200, 150, 64], np.int32)
    cache, kd, vd = fill_stream_cache(dev, B, n_kv, ctx, lens, 5, bits=bits, symmetric=(bits == 8), shift=0.0 if bits == 8 else 0.5)
    segs = B * n_kv if per_head else B
    rng = np.random.default_rng(0)
    acc = rng.random((segs, ctx)).astype(F32)
    ts = np.tile(np.arange(ctx, dtype=F32), (segs, 1))
    seg_len = np.repeat(lens, n_kv) if per_head else lens
    mask, keep, cnt = ops.h2o_select(torch.from_numpy(acc).to(dev), torch.from_numpy(ts).to(dev), 40, 8,
                                     seg_len=torch.from_numpy(seg_len.astype(np.int32)).to(dev))
    dst = pikv_b200.PagedKVCache(B, ctx, n_kv, bits=bits, symmetric=(bits == 8), device=dev)
    # destination score rows as long as the source's, or only as long as the kept-index rows
    width = keep.shape[1] if per_head else ctx
    dacc = torch.zeros(segs, width, device=dev)
    dts = torch.zeros(segs, width, device=dev)
    guard = torch.zeros(1 << 16, device=dev)          # allocated right after them: must stay untouched
    cache.compact_into(dst, keep, cnt, per_head, torch.from_numpy(acc).to(dev), torch.from_numpy(ts).to(dev), dacc, dts)
    cache.check_status()
    assert float(guard.abs().sum()) == 0.0
    with pytest.raises(pikv_b200.PikvError):
        cache.compact_into(dst, keep, cnt, per_head, torch.from_numpy(acc).to(dev), torch.from_numpy(ts).to(dev),
                           dacc[:, : keep.shape[1] - 1].contiguous(), dts[:, : keep.shape[1] - 1].contiguous())
    for s in range(segs):
        b = s // n_kv if per_head else s
        heads = [s % n_kv] if per_head else list(range(n_kv))
        ev, ki = O.h2o_select(acc[s, : seg_len[s]], ts[s, : seg_len[s]], 40, 8)
        n = len(ki)
        seq = torch.full((n,), b, dtype=torch.int32, device=dev)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        gk = dst.gather(seq, pos, "k").cpu().numpy().reshape(n, n_kv, 128)
        gv = dst.gather(seq, pos, "v").cpu().numpy().reshape(n, n_kv, 128)
        for h in heads:
            np.testing.assert_array_equal(gk[:, h], kd[b, h, ki])
            np.testing.assert_array_equal(gv[:, h], vd[b, h, ki])
        np.testing.assert_array_equal(dacc[s, :n].cpu().numpy(), acc[s, ki])
        np.testing.assert_array_equal(dts[s, :n].cpu().numpy(), ts[s, ki])


# ---------------------------------------------------------------- exchange records
def test_a2a_pack_unpack_equals_direct_append(dev):
    import pikv_b200
    from pikv_b200 import ops
    T, E, k, n_kv = 500, 4, 2, 2
    K, V = outlier_kv(T, n_kv * 128, 8).to(dev), outlier_kv(T, n_kv * 128, 9).to(dev)
    rng = np.random.default_rng(4)
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    cap = 300
    slot, _ = O.slot_assign_fast(idx, E, cap)
    direct = pikv_b200.PagedKVCache(E, cap, n_kv, device=dev)
    direct.append(K, V, torch.from_numpy(idx).to(dev), torch.from_numpy(slot).to(dev))
    # records in (destination, token, j) order, as the exchange would deliver them
    flat_ok = (slot >= 0).reshape(-1)
    order = np.argsort(idx.reshape(-1) // 2, kind="stable")            # two "ranks" own two experts each
    order = order[flat_ok[order]]
    send_pos = np.full(T * k, -1, np.int32)
    send_pos[order] = np.arange(len(order), dtype=np.int32)
    buf = ops.a2a_pack(K, V, n_kv, torch.from_numpy(idx).to(dev), torch.from_numpy(slot).to(dev), len(order),
                       send_pos=torch.from_numpy(send_pos.reshape(T, k)).to(dev))
    via = pikv_b200.PagedKVCache(E, cap, n_kv, device=dev)
    via.unpack_records(buf, len(order))
    via.check_status()
    for name in ("k_codes", "v_codes", "k_scale", "v_scale"):
        assert torch.equal(getattr(direct, name), getattr(via, name)), name


def test_sharded_cache_single_rank_equals_direct_append(dev):
    """World size 1: gate -> pack -> (no exchange) -> unpack must leave exactly the cache the direct
    route + append leaves."""
    import pikv_b200
    from pikv_b200 import ops
    from pikv_b200.distributed import ExpertShardedKVCache
    T, H, E, k, n_kv, cap = 3000, 512, 8, 2, 2, 700          # capacity forces drops on the owner side
    torch.manual_seed(3)
    act = torch.randn(T, H, device=dev).bfloat16()
    w2 = (torch.randn(E, H, device=dev) / 20).bfloat16()
    K, V = outlier_kv(T, n_kv * 128, 5).to(dev), outlier_kv(T, n_kv * 128, 6).to(dev)
    g = ops.gate_fused(act, w2, None, top_k=k, capacity=cap)
    direct = pikv_b200.PagedKVCache(E, cap, n_kv, device=dev)
    direct.append(K, V, g.topk_idx, g.slot)
    shard = ExpertShardedKVCache(E, cap, n_kv, dev)
    shard.route_append(act, w2, None, K, V, top_k=k)
    shard.cache.check_status()
    for name in ("k_codes", "v_codes", "k_scale", "v_scale"):
        assert torch.equal(getattr(direct, name), getattr(shard.cache, name)), name
    assert torch.equal(shard.cache.length, g.new_len)


@pytest.mark.parametrize("T,H,E,k,n_kv,cap", [(16384, 4096, 8, 2, 8, 6144), (3000, 512, 8, 2, 2, 700), (129, 256, 64, 4, 1, 40),
                                              (70000, 128, 16, 1, 1, 0)])
def test_fused_route_append_equals_gate_then_append(dev, T, H, E, k, n_kv, cap):
    """pikv_route_append (slot finalisation folded into the append kernel) against the two separate
    entry points: slots, counts, lengths, probabilities and every byte of the cache."""
    import pikv_b200
    from pikv_b200 import ops
    torch.manual_seed(T)
    act = torch.relu(torch.randn(T, H, device=dev)).bfloat16()
    w2 = (torch.randn(E, H, device=dev) / H ** 0.5).bfloat16()
    b2 = torch.randn(E, device=dev) * 0.1
    K, V = outlier_kv(T, n_kv * 128, 5).to(dev), outlier_kv(T, n_kv * 128, 6).to(dev)
    size = cap if cap > 0 else T
    base = torch.randint(0, 5, (E,), dtype=torch.int32, device=dev)
    g = ops.gate_fused(act, w2, b2, top_k=k, capacity=cap, slot_base=base)
    two = pikv_b200.PagedKVCache(E, size + 8, n_kv, device=dev)
    two.append(K, V, g.topk_idx, g.slot)
    one = pikv_b200.PagedKVCache(E, size + 8, n_kv, device=dev)
    f = one.route_append(act, w2, b2, K, V, top_k=k, capacity=cap, slot_base=base)
    one.check_status()
    assert torch.equal(f.topk_idx, g.topk_idx) and torch.equal(f.slot, g.slot)
    assert torch.equal(f.counts_k, g.counts_k) and torch.equal(f.new_len, g.new_len)
    assert torch.equal(f.probs, g.probs) and torch.equal(f.topk_w, g.topk_w)
    assert torch.allclose(f.prob_sum, g.prob_sum, rtol=1e-5)
    for name in ("k_codes", "v_codes", "k_scale", "v_scale"):
        assert torch.equal(getattr(one, name), getattr(two, name)), name



def test_cache_checkpoint_round_trip(dev):
    """The cache's state (pages, scales, page table, lengths) travels through state_dict / torch.save and
    decodes to the same bits afterwards (the reference checkpoints only a mean vector per expert,
    core/single/pikv_moe.py:456-505)."""
    import io
    import pikv_b200
    B, n_q, n_kv, ctx = 3, 8, 2, 300
    lens = np.array([300, 17, 160], np.int32)
    cache, _, _ = fill_stream_cache(dev, B, n_kv, ctx, lens, 21)
    q = torch.randn(B, n_q, 128, device=dev).bfloat16()
    want = cache.decode_attention(q, splits=2)
    buf = io.BytesIO()
    torch.save(cache.state_dict(), buf)
    buf.seek(0)
    fresh = pikv_b200.PagedKVCache(B, ctx, n_kv, device=dev)
    fresh.load_state_dict(torch.load(buf, map_location=dev))
    assert torch.equal(fresh.page_table, cache.page_table) and torch.equal(fresh.length, cache.length)
    assert torch.equal(fresh.decode_attention(q, splits=2), want)


def test_other_eviction_policies_match_reference(dev):
    """StreamingLLM / LRU / LRU+ / FlexGen / QUEST select_eviction_candidates against the reference's masks
    (tie-free buffers); the lowest-m choice runs on the segmented select kernel."""
    import pikv_b200
    g = load_golden("eviction_policies")
    C, H, n = 48, 8, 64
    keys = torch.from_numpy(g["keys"]).to(dev)

    def t(name):
        return torch.from_numpy(g[name]).to(dev)

    st = pikv_b200.StreamingLLMScheduler(C, H, start_size=4, recent_size=20).to(dev)
    np.testing.assert_array_equal(st.select_eviction_candidates(keys, keys, {}).cpu().numpy(), g["streaming/mask"])
    np.testing.assert_array_equal(st.select_eviction_candidates(keys[:40], keys[:40], {}).cpu().numpy(), g["streaming/small"])
    lru = pikv_b200.LRUScheduler(C, H).to(dev)
    lru.access_times.copy_(t("lru/access_times"))
    before = pikv_b200.launch_count()
    np.testing.assert_array_equal(lru.select_eviction_candidates(keys, keys, {}).cpu().numpy(), g["lru/mask"])
    assert pikv_b200.launch_count() > before
    lp = pikv_b200.LRUPlusScheduler(C, H).to(dev)
    for k in ("access_times", "access_frequency", "importance_scores"):
        getattr(lp, k).copy_(t(f"lru_plus/{k}"))
    assert np.abs(lp.compute_priority_scores(n).cpu().numpy() - g["lru_plus/priority"]).max() < 1e-6
    np.testing.assert_array_equal(lp.select_eviction_candidates(keys, keys, {}).cpu().numpy(), g["lru_plus/mask"])
    fg = pikv_b200.FlexGenScheduler(C, H).to(dev)
    fg.access_frequency.copy_(t("flexgen/access_frequency"))
    fg.access_cost.copy_(t("flexgen/access_cost"))
    np.testing.assert_array_equal(fg.select_eviction_candidates(keys, keys, {}).cpu().numpy(), g["flexgen/mask"])
    for tag, thr in (("few", 0.001), ("many", 5.0)):
        q = pikv_b200.QUESTScheduler(C, H, quality_threshold=thr).to(dev)
        for k in ("quality_scores", "usage_frequency", "last_access_time"):
            getattr(q, k).copy_(t(f"quest_{tag}/{k}"))
        q.global_time.fill_(C)
        np.testing.assert_array_equal(q.select_eviction_candidates(keys, keys, {}).cpu().numpy(), g[f"quest_{tag}/mask"])
    # update methods run (the reference's LRU one raises under this torch: it stores an int64 time into a float
    # buffer) and the manager with such a policy fills up and stops
    lru.update_access_time(torch.tensor([1, 2], device=dev))
    assert float(lru.access_times[1]) == 0.0 and int(lru.global_time) == 1
    mgr = pikv_b200.CacheSchedulingManager(16, H, pikv_b200.SchedulingPolicy.LRU).to(dev)
    for i in range(3):
        mgr.update_cache(keys[None, 7 * i: 7 * i + 7], keys[None, 7 * i: 7 * i + 7])
    assert int(mgr.cache_size_current) == int(g["manager_lru/size"])
    np.testing.assert_array_equal(mgr.cache_keys.cpu().numpy(), g["manager_lru/keys"])


def test_module_adakv_and_duo_attention_match_reference(dev):
    """AdaKVScheduler / DuoAttentionScheduler (core/single/module/pikv_scheduling.py:624-710) against the
    reference's masks; both run on the segmented select kernel."""
    import pikv_b200
    from pikv_b200.module import AdaKVScheduler, DuoAttentionScheduler
    g = load_golden("eviction_policies_module")
    C, H, n = 48, 8, 64
    keys = torch.from_numpy(g["keys"]).to(dev)
    ada = AdaKVScheduler(C, H, compression_ratio=0.5, safeguard_ratio=0.2).to(dev)
    ada.linear_proj.weight.data.copy_(torch.from_numpy(g["adakv/weights/weight"]))
    ada.linear_proj.bias.data.copy_(torch.from_numpy(g["adakv/weights/bias"]))
    with torch.no_grad():
        ada.update_importance(torch.arange(C, device=dev), keys[:C])
    assert np.abs(ada.importance_scores.cpu().numpy() - g["adakv/importance_scores"]).max() < 1e-5
    ada.importance_scores.copy_(torch.from_numpy(g["adakv/importance_scores"]))
    before = pikv_b200.launch_count()
    np.testing.assert_array_equal(ada.select_eviction_candidates(keys, keys, {}).cpu().numpy(), g["adakv/mask"])
    assert pikv_b200.launch_count() > before
    np.testing.assert_array_equal(ada.select_eviction_candidates(keys[:40], keys[:40], {}).cpu().numpy(), g["adakv/small"])
    duo = DuoAttentionScheduler(C, H, sink_size=5, recent_size=17).to(dev)
    np.testing.assert_array_equal(duo.select_eviction_candidates(keys, keys, {}).cpu().numpy(), g["duo/mask"])
    np.testing.assert_array_equal(duo.select_eviction_candidates(keys[:40], keys[:40], {}).cpu().numpy(), g["duo/small"])
    assert int(duo.eviction_count) == int(g["duo/evictions"])
    assert duo.get_scheduler_stats()["sink_size"] == 5


def test_append_rope_matches_reference(dev):
    """Rotary embedding + quantise + append in one kernel: K codes and scales equal the oracle's quantisation of
    the reference's rotated keys (golden fixture from RotaryEmbedding.forward), bit for bit; V as the plain append."""
    import pikv_b200
    g = load_golden("rope")
    cos, sin = torch.from_numpy(g["cos"]).to(dev), torch.from_numpy(g["sin"]).to(dev)
    k = torch.from_numpy(g["k"]).reshape(48, 3 * 128)                         # [B*S, heads*128], bf16-valued
    pos = torch.from_numpy(g["positions"].reshape(-1).astype(np.int32))
    v = torch.randn(48, 3 * 128).bfloat16()
    cache = pikv_b200.PagedKVCache(2, 40, 3, device=dev)
    dst = torch.arange(48, dtype=torch.int32)[:, None] % 2
    slot = (torch.arange(48, dtype=torch.int32)[:, None] // 2).contiguous()
    cache.append_rope(k.bfloat16().to(dev), v.to(dev), dst.to(dev).contiguous(), slot.to(dev), cos, sin, pos.to(dev))
    torch.cuda.synchronize()
    cache.check_status()
    want_k = g["k_out"].reshape(48, 3 * 128)                                  # the reference's rotated keys
    q, sc, _ = O.quant_token_groups(want_k, 8, 128, True)
    dq, codes = cache.gather(dst[:, 0].to(dev).contiguous(), slot[:, 0].to(dev).contiguous(), "k", codes=True)
    np.testing.assert_array_equal(codes.cpu().numpy().astype(F32), q)
    np.testing.assert_array_equal(dq.cpu().numpy(), O.dequant_token_groups(q, O.bf16_round(sc), np.zeros_like(sc), 128))
    qv, _, _ = O.quant_token_groups(v.float().numpy(), 8, 128, True)
    _, vcodes = cache.gather(dst[:, 0].to(dev).contiguous(), slot[:, 0].to(dev).contiguous(), "v", codes=True)
    np.testing.assert_array_equal(vcodes.cpu().numpy().astype(F32), qv)
    # positions default to the token index
    cache2 = pikv_b200.PagedKVCache(1, 48, 3, device=dev)
    s2 = torch.arange(48, dtype=torch.int32, device=dev)[:, None].contiguous()
    cache2.append_rope(k.bfloat16().to(dev), v.to(dev), torch.zeros_like(s2), s2, cos, sin)
    want2 = O.rope_rotate(g["k"].reshape(48, 3, 128), np.arange(48), g["cos"], g["sin"]).reshape(48, 384)
    q2, _, _ = O.quant_token_groups(want2, 8, 128, True)
    _, c2 = cache2.gather(torch.zeros(48, dtype=torch.int32, device=dev), s2[:, 0].contiguous(), "k", codes=True)
    np.testing.assert_array_equal(c2.cpu().numpy().astype(F32), q2)


def test_cache_checkpoint_round_trip(dev, tmp_path):
    """Pages, scales, zero points, page table, lengths and a policy's score buffers survive save / load: the
    reloaded cache decodes to the same bits (the reference's checkpoint keeps one mean vector per cache)."""
    import pikv_b200
    for bits in (8, 4):
        B, n_kv, ctx = 3, 2, 200
        lens = np.array([200, 150, 64], np.int32)
        cache, _, _ = fill_stream_cache(dev, B, n_kv, ctx, lens, 11, bits=bits, symmetric=(bits == 8))
        acc = torch.rand(B * n_kv, ctx, device=dev)
        path = tmp_path / f"cache{bits}.pt"
        cache.save_checkpoint(path, scores={"attention_accumulator": acc})
        again, scores = pikv_b200.PagedKVCache.load_checkpoint(path, device=dev)
        assert torch.equal(scores["attention_accumulator"], acc)
        for name in ("k_codes", "v_codes", "k_scale", "v_scale", "page_table", "length") + (("k_zp", "v_zp") if bits == 4 else ()):
            assert torch.equal(getattr(again, name), getattr(cache, name)), name
        q = torch.randn(B, 4 * n_kv, 128, device=dev).bfloat16()
        assert torch.equal(again.decode_attention(q), cache.decode_attention(q))
