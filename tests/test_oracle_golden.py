"""The numpy oracle against vectors produced by the reference's own modules."""
import math

import numpy as np
import pytest

from conftest import load_golden, sub
from oracle import pikv_oracle as O

F32 = np.float32


def mlp(x, w, prefix, n=2):
    h = x @ w[f"{prefix}.0.weight"].T + w[f"{prefix}.0.bias"]
    h = np.maximum(h, 0)
    last = max(int(k.split(".")[-2]) for k in w if k.startswith(prefix + ".") and k.endswith("weight"))
    return h @ w[f"{prefix}.{last}.weight"].T + w[f"{prefix}.{last}.bias"]


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def close(a, b, rtol=1e-5, atol=1e-6):
    np.testing.assert_allclose(np.asarray(a, np.float64), np.asarray(b, np.float64), rtol=rtol, atol=atol)


# ---------------------------------------------------------------- routers
def test_base_router_single():
    g = load_golden("router_base_single")
    w = sub(g, "weights")
    x = g["x"].reshape(-1, 64)
    logits = O.gate_logits(np.maximum(x @ w["router.0.weight"].T + w["router.0.bias"], 0),
                           w["router.2.weight"], w["router.2.bias"])
    close(logits, g["logits"].reshape(-1, 4), 1e-4, 1e-5)
    for tag, mask in (("", None), ("_m", g["mask"])):
        probs, idx, tw = O.gate_tail(g["logits"].reshape(-1, 4), 2, expert_mask=mask, mask_mode="single")
        close(probs, g["probs" + tag].reshape(-1, 4))
        cap = O.capacity(32, 1.5, 2, 4)
        d, c = O.dispatch_combine_single(idx, tw, 4, cap)
        np.testing.assert_array_equal(d, g["dispatch" + tag].reshape(32, 4, cap))
        close(c, g["combine" + tag].reshape(32, 4, cap))
        close(O.aux_loss_base(probs, 4), g["aux" + tag], 1e-4, 1e-6)
        # every routed (token, expert) pair appears exactly once in the dense tensor
        assert d.sum() == 64


def test_topk_balanced_single():
    g = load_golden("router_topk_balanced_single")
    x = g["x"].reshape(-1, 64)
    for mode in ("entropy", "cv", "l2"):
        s = sub(g, mode)
        w = sub(s, "weights")
        probs, idx, tw = O.gate_tail(mlp(x, w, "router"), 2)
        close(probs, s["probs"].reshape(-1, 4), 1e-4, 1e-6)
        close(O.aux_loss_topk_balanced(probs, 4, 0.01, mode), s["aux"], 1e-4, 1e-6)


def test_pikv_router_single_state_machine():
    g = load_golden("router_pikv_single")
    w = sub(g, "weights")
    hist = w["cache_usage_history"].copy()
    factor = w["cache_correction_factor"].copy()
    counter = int(w["update_counter"])
    for i in range(3):
        c = sub(g, f"call{i}")
        x = c["x"].reshape(-1, 64)
        imp = sigmoid(mlp(x, w, "importance_predictor"))
        if i == 1:
            imp = (imp + sigmoid(mlp(g["kv"].reshape(-1, 64), w, "kv_importance_model"))) / 2
        close(imp, c["importance"].reshape(-1, 1), 1e-5, 1e-6)
        m = (imp > 0.5).astype(F32)
        logits = m * mlp(x, w, "router_important") + (1 - m) * mlp(x, w, "router_unimportant")
        probs, idx, tw = O.gate_tail(logits.astype(F32), 2, correction=factor)
        close(probs, c["probs"].reshape(-1, 4), 1e-4, 1e-6)
        usage = probs.sum(axis=0)
        usage = usage / usage.sum()
        hist = 0.9 * hist + 0.1 * usage                       # pikv_routing.py:419
        counter += 1
        if counter % 2 == 0:                                  # :425-430
            factor = 1.0 / (hist + 0.5)
            factor = factor / factor.mean()
        close(hist, c["history"], 1e-5, 1e-7)
        close(factor, c["factor"], 1e-5, 1e-7)
        aux = O.aux_loss_base(probs, 4) + 0.05 * np.sum(hist * usage)
        close(aux, c["aux"], 1e-4, 1e-6)
        cap = O.capacity(32, 1.5, 2, 4)
        d, cmb = O.dispatch_combine_single(idx, tw, 4, cap)
        np.testing.assert_array_equal(d, c["dispatch"].reshape(32, 4, cap))
        close(cmb, c["combine"].reshape(32, 4, cap))


def test_base_router_module_running_slots():
    g = load_golden("router_base_module")
    probs, idx, tw = O.gate_tail(g["logits"].reshape(-1, 4), 2, renorm_eps=1e-8)
    close(probs, g["probs"].reshape(-1, 4))
    cap = O.capacity(24, 1.0, 2, 4)
    d, c = O.dispatch_combine_module(idx, tw, 4, cap)
    np.testing.assert_array_equal(d, g["dispatch"].reshape(24, 4, cap))
    close(c, g["combine"].reshape(24, 4, cap))
    close(O.aux_loss_module(probs, idx, 4), g["aux"], 1e-5, 1e-6)
    slot, counts_k = O.slot_assign(idx, 4, cap)
    np.testing.assert_array_equal(counts_k.sum(0), g["usage"].astype(np.int64))
    s2, c2 = O.slot_assign_fast(idx, 4, cap)
    np.testing.assert_array_equal(slot, s2)
    np.testing.assert_array_equal(counts_k, c2)
    # capacity_factor 1.0 forces drops: dropped pairs have slot -1 and no dispatch entry
    assert (slot < 0).sum() == 48 - int(d.sum())


def _module_router_tail(g, w, logits, k, importance=None, threshold=None):
    x = g["x"]
    tokens = x.shape[0] * x.shape[1]
    probs, idx, tw = O.gate_tail(logits.reshape(-1, 4), k, renorm_eps=1e-8)
    close(probs, g["probs"].reshape(-1, 4))
    cap = O.capacity(tokens, 1.5, k, 4)
    d, c = O.dispatch_combine_module(idx, tw, 4, cap)
    if importance is not None:
        c = c * (1.0 + (importance.reshape(-1) > threshold).astype(F32))[:, None, None]
    np.testing.assert_array_equal(d, g["dispatch"].reshape(tokens, 4, cap))
    close(c, g["combine"].reshape(tokens, 4, cap))
    close(O.aux_loss_module(probs, idx, 4), g["aux"], 1e-5, 1e-6)
    _, counts_k = O.slot_assign(idx, 4, cap)
    np.testing.assert_array_equal(counts_k.sum(0), g["usage"].astype(np.int64))


def test_module_pikv_router():
    g = load_golden("router_pikv_module")
    w = sub(g, "weights")
    x = g["x"]
    imp = sigmoid(mlp(x, w, "importance_predictor"))[..., 0]
    close(imp, g["importance"])
    k = O.module_adaptive_top_k(x, imp, w["top_k_predictor.0.weight"], w["top_k_predictor.0.bias"],
                                w["top_k_predictor.2.weight"], w["top_k_predictor.2.bias"], 2)
    adj = O.module_cache_adjustment(x, w["cache_hit_rates"], w["cache_router_adjustment.0.weight"],
                                    w["cache_router_adjustment.0.bias"], w["cache_router_adjustment.2.weight"],
                                    w["cache_router_adjustment.2.bias"])
    logits = mlp(x, w, "router") + adj[:, None, :]
    _module_router_tail(g, w, logits, k)


def test_module_adaptive_router():
    g = load_golden("router_adaptive_module")
    w = sub(g, "weights")
    x = g["x"]
    imp = sigmoid(mlp(x, w, "importance_predictor"))[..., 0]
    close(imp, g["importance"])
    k = O.module_adaptive_top_k(x, imp, w["top_k_predictor.0.weight"], w["top_k_predictor.0.bias"],
                                w["top_k_predictor.2.weight"], w["top_k_predictor.2.bias"], 2)
    _module_router_tail(g, w, mlp(x, w, "router"), k, imp, 0.5)
    n = imp.size
    close(g["history"][:n], imp.reshape(-1))
    assert int(g["history_idx"]) == n


def test_module_pyramid():
    g = load_golden("pyramid_module")
    w = sub(g, "weights")
    levels = O.module_pyramid_levels(g["importance"], w["importance_thresholds"])
    np.testing.assert_array_equal(levels, g["levels"])
    layers = [dict(enc_w=w[f"compression_layers.{i}.encoder.0.weight"], enc_b=w[f"compression_layers.{i}.encoder.0.bias"],
                   enc_g=w[f"compression_layers.{i}.encoder.1.weight"], enc_beta=w[f"compression_layers.{i}.encoder.1.bias"],
                   dec_w=w[f"compression_layers.{i}.decoder.0.weight"], dec_b=w[f"compression_layers.{i}.decoder.0.bias"],
                   dec_g=w[f"compression_layers.{i}.decoder.1.weight"], dec_beta=w[f"compression_layers.{i}.decoder.1.bias"])
              for i in range(3)]
    close(O.module_pyramid(g["keys"].reshape(-1, 64), levels.reshape(-1), layers), g["ck"].reshape(-1, 64), 1e-4, 1e-5)
    uniform = O.module_pyramid_levels(np.full((2, 10), 0.5, F32), w["importance_thresholds"])
    close(O.module_pyramid(g["values"].reshape(-1, 64), uniform.reshape(-1), layers), g["nv"].reshape(-1, 64), 1e-4, 1e-5)


def test_strategy_adaptive_router():
    g = load_golden("router_strategy_adaptive")
    w = sub(g, "weights")
    x = g["x"]
    x2 = x.reshape(-1, 64)
    lb_w, lb_i, lb_t = O.gate_tail(mlp(x2, w, "load_balancing_router.router"), 2)
    close(lb_w, g["lb_weights"].reshape(-1, 4), 1e-4, 1e-6)
    np.testing.assert_array_equal(lb_i, g["lb_indices"].reshape(-1, 2))
    imp = sigmoid(mlp(x2, w, "importance_router.importance_predictor"))
    iw, _, _ = O.gate_tail(mlp(x2, w, "importance_router.router"), 2)
    iw = iw * imp
    iw = iw / iw.sum(-1, keepdims=True)
    sel = O.softmax_f32(mlp(x.mean(1), w, "router_selector"))           # routing_strategy.py:133-134
    sel_tok = np.repeat(sel, x.shape[1], axis=0)
    rw = sel_tok[:, 0:1] * lb_w + sel_tok[:, 1:2] * iw
    close(rw, g["routing_weights"].reshape(-1, 4), 1e-4, 1e-6)
    tv, ti = O.stable_topk(rw, 2)
    np.testing.assert_array_equal(ti, g["expert_indices"].reshape(-1, 2))
    close(tv / tv.sum(-1, keepdims=True), g["top_k_weights"].reshape(-1, 2), 1e-4, 1e-6)
    usage = lb_w.mean(0)
    close(0.01 * usage.std(ddof=1) / usage.mean(), g["lb_loss"], 1e-4, 1e-7)


# ---------------------------------------------------------------- quantisation
@pytest.mark.parametrize("tag,bits,gs,sym", [
    ("single_b8g1", 8, 1, False), ("single_b4g16", 4, 16, False), ("single_b8g64", 8, 64, False),
    ("module_b8g32s", 8, 32, True), ("module_b4g32a", 4, 32, False), ("module_b4g16s", 4, 16, True),
    ("module_b8g64a", 8, 64, False)])
def test_quant_block_bit_exact(tag, bits, gs, sym):
    g = load_golden("quant_block")
    for name in ("keys", "values"):
        x = g[name].reshape(-1, 64)
        dq, q, sc, zp, mse = O.quant_block_forward(x, bits, gs, sym)
        np.testing.assert_array_equal(dq, g[f"{tag}/dq_{name}"].reshape(-1, 64))
    close(mse, g[f"{tag}/quantization_error"], 1e-5, 1e-9)


def test_quant_slices_bit_exact():
    g = load_golden("quant_slices")
    x = g["x"]
    for tag, bits, sym in (("int8_sym", 8, True), ("int4_asym", 4, False), ("int8_asym", 8, False),
                           ("int4_sym", 4, True)):
        q, sc, zp = O.quant_token_groups(x, bits, 128, sym)
        np.testing.assert_array_equal(q, g[f"{tag}/q"])
        np.testing.assert_array_equal(sc, g[f"{tag}/scale"])
        np.testing.assert_array_equal(O.dequant_token_groups(q, sc, zp, 128), g[f"{tag}/dq"])


# ---------------------------------------------------------------- H2O
def test_h2o_select_matches_reference_mask():
    g = load_golden("h2o_select")
    n = int(g["n"])
    nh, nr = O.h2o_counts(n, 0.1, 0.05)
    evict, keep = O.h2o_select(g["acc"][:n], g["ts"][:n], nh, nr)
    np.testing.assert_array_equal(evict, g["evict_mask"])
    assert np.all(np.diff(keep) > 0)
    assert int(g["update_raises"]) == 1     # the reference's accumulate step raises under this torch


def test_h2o_ties_lowest_index():
    acc = np.array([1, 3, 3, 3, 0, 3], F32)
    ts = np.arange(6, dtype=F32)
    evict, keep = O.h2o_select(acc, ts, 2, 1)
    np.testing.assert_array_equal(keep, [1, 2, 5])


def test_eviction_policies():
    g = load_golden("eviction_policies")
    C, n = 48, 64
    np.testing.assert_array_equal(O.streaming_llm_mask(n, C, 4, 20), g["streaming/mask"])
    np.testing.assert_array_equal(O.streaming_llm_mask(40, C, 4, 20), g["streaming/small"])
    np.testing.assert_array_equal(O.evict_lowest(g["lru/access_times"], n - C, n), g["lru/mask"])
    pr = O.lru_plus_priority(g["lru_plus/access_times"], g["lru_plus/access_frequency"], g["lru_plus/importance_scores"])
    close(pr, g["lru_plus/priority"])
    np.testing.assert_array_equal(O.evict_lowest(pr, n - C, n), g["lru_plus/mask"])
    np.testing.assert_array_equal(O.evict_lowest(g["flexgen/access_frequency"] / g["flexgen/access_cost"], n - C, n),
                                  g["flexgen/mask"])
    for tag, thr in (("few", 0.001), ("many", 5.0)):
        u = O.quest_utility(g[f"quest_{tag}/quality_scores"], g[f"quest_{tag}/usage_frequency"],
                            g[f"quest_{tag}/last_access_time"], C)
        close(u, g[f"quest_{tag}/utility"])
        np.testing.assert_array_equal(O.quest_mask(u, thr, n, C), g[f"quest_{tag}/mask"])
    # through the manager the cache only fills up: 16 of the 21 offered rows, in order
    assert int(g["manager_lru/size"]) == 16
    np.testing.assert_array_equal(g["manager_lru/keys"], g["keys"][:16])


def test_h2o_manager_sequence():
    g = load_golden("h2o_manager")
    ck = np.zeros((64, 8), F32)
    cv = np.zeros((64, 8), F32)
    size, evictions = 0, 0
    for s in range(5):
        c = sub(g, f"s{s}")

        def evict_fn(n, c=c):
            nh, nr = O.h2o_counts(n, 0.1, 0.1)
            return O.h2o_select(c["acc"][:n], c["ts"][:n], nh, nr)[0]

        size, ev = O.manager_update_cache(ck, cv, size, c["keys_in"], c["values_in"], evict_fn)
        evictions += ev
        assert size == int(c["size"])
        assert evictions == int(c["evictions"])
        np.testing.assert_array_equal(ck[:size], c["cache_keys"][:size])
        np.testing.assert_array_equal(cv[:size], c["cache_values"][:size])


# ---------------------------------------------------------------- attention / projection
def test_decode_attention_matches_reference_mha():
    g = load_golden("attention_decode")
    q = g["q"][:, 0]                                   # [B, heads, d]
    k = np.transpose(g["k"], (0, 2, 1, 3))             # [B, heads, ctx, d]
    v = np.transpose(g["v"], (0, 2, 1, 3))
    out, psum = O.decode_attention(q, k, v)
    close(out, g["context"][:, 0], 1e-5, 1e-6)
    close(psum.sum(-1), np.ones_like(psum.sum(-1)), 1e-5)


def test_lowrank_svd():
    g = load_golden("lowrank_svd_single")
    w = sub(g, "weights")
    for n, p in (("keys", "key"), ("values", "value")):
        x = g[n].reshape(-1, 64)
        y = O.lowrank_project(x, w[f"{p}_projector.weight"], w[f"{p}_projector.bias"])
        rec = O.lowrank_reconstruct(y, w[f"{p}_reconstructor.weight"], w[f"{p}_reconstructor.bias"])
        close(rec, g[f"rec_{n}"].reshape(-1, 64), 1e-4, 1e-5)
    g = load_golden("lowrank_svd_module")
    w = sub(g, "weights")
    r = int(g["effective_rank"])
    assert 1 <= r < 16
    for n, p in (("keys", "key"), ("values", "value")):
        rec = O.svd_compress(g[n].reshape(-1, 64), w[f"{p}_projector.weight"], w[f"{p}_projector.bias"],
                             w[f"{p}_reconstructor.weight"], w[f"{p}_reconstructor.bias"], rank_keep=r, pad=True)
        close(rec, g[f"rec_{n}"].reshape(-1, 64), 1e-4, 1e-5)


def test_pyramid():
    g = load_golden("pyramid_single")
    w = sub(g, "weights")
    enc = [(w[f"encoder_layers.{i}.weight"], w[f"encoder_layers.{i}.bias"]) for i in range(3)]
    dec = [(w[f"decoder_layers.{i}.weight"], w[f"decoder_layers.{i}.bias"]) for i in range(3)]
    for n in ("keys", "values"):
        x = g[n].reshape(-1, 64)
        close(O.pyramid_uniform(x, enc, dec), g[f"uni_{n}"].reshape(-1, 64), 1e-4, 1e-5)
        close(O.pyramid_importance(x, g["importance"].reshape(-1), enc, dec, 3, 0.8),
              g[f"imp_{n}"].reshape(-1, 64), 1e-4, 1e-5)
    g = load_golden("cache_pyramid")
    w = sub(g, "weights")
    args = (w["compressor.compression_layers.0.weight"], w["compressor.compression_layers.0.bias"],
            w["compressor.compression_layers.1.weight"], w["compressor.compression_layers.1.bias"])
    close(O.cache_pyramid_compression(g["keys"], g["importance"], *args), g["ck"], 1e-4, 1e-5)
    close(O.cache_pyramid_compression(g["values"], None, *args), g["nv"], 1e-4, 1e-5)


def test_bf16_round():
    import torch
    x = np.random.default_rng(0).standard_normal(10000).astype(F32) * 37
    ref = torch.from_numpy(x).bfloat16().float().numpy()
    np.testing.assert_array_equal(O.bf16_round(x), ref)


def test_module_adakv_and_duo_attention_masks():
    g = load_golden("eviction_policies_module")
    C, n = 48, 64
    sc = g["adakv/importance_scores"]
    np.testing.assert_array_equal(O.adakv_mask(sc, n, C, 0.5), g["adakv/mask"])
    np.testing.assert_array_equal(O.adakv_mask(sc, 40, C, 0.5), g["adakv/small"])
    np.testing.assert_array_equal(O.duo_attention_mask(n, C, 5, 17), g["duo/mask"])
    np.testing.assert_array_equal(O.duo_attention_mask(40, C, 5, 17), g["duo/small"])
    assert int(g["duo/evictions"]) == 1


def test_rope_matches_reference():
    g = load_golden("rope")
    for b in range(2):
        np.testing.assert_array_equal(O.rope_rotate(g["q"][b], g["positions"][b], g["cos"], g["sin"]), g["q_out"][b])
        np.testing.assert_array_equal(O.rope_rotate(g["k"][b], g["positions"][b], g["cos"], g["sin"]), g["k_out"][b])
    c, s_ = O.rope_tables(96, 128)
    assert np.abs(c - g["cos"]).max() < 1e-5 and np.abs(s_ - g["sin"]).max() < 1e-5     # fp32 angles up to 95 rad
