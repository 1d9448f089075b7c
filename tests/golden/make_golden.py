"""Generate golden input/output vectors by running the reference's own modules.

Run where the reference project is checked out:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <path>

It imports the reference's PyTorch operators (CPU), feeds them seeded inputs
and stores inputs, weights and outputs as small .npz files next to this
script.  The test-suite then checks the numpy oracle and the CUDA kernels
against these files on machines that do not have the reference.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def npy(t):
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().numpy()
    return np.asarray(t)


def sd(module):
    return {k: npy(v).copy() for k, v in module.state_dict().items()}


ONLY = None      # --only NAME: write just that fixture (the others are recomputed but left alone)


def save(name, **arrays):
    if ONLY is not None and name != ONLY:
        return
    flat = {}
    for k, v in arrays.items():
        if isinstance(v, dict):
            for kk, vv in v.items():
                flat[f"{k}/{kk}"] = npy(vv)
        else:
            flat[k] = npy(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **flat)
    print(f"{name}: {len(flat)} arrays")


def router_fixtures(ref_single, ref_module, ref_strategy):
    # R1/R2: core/single BaseRouter + TopKBalancedRouter (3 balance modes)
    torch.manual_seed(0)
    H, E, K = 64, 4, 2
    x = torch.randn(2, 16, H)
    mask = torch.tensor([1.0, 1.0, 0.0, 1.0])
    r = ref_single.BaseRouter(H, E, K)
    with torch.no_grad():
        logits = r.router(x)
        act = r.router[1](r.router[0](x))
        d, c, p, aux = r(x)
        dm, cm, pm, auxm = r(x, mask)
    save("router_base_single", x=x, act=act, logits=logits, mask=mask, weights=sd(r),
         dispatch=d, combine=c, probs=p, aux=aux, dispatch_m=dm, combine_m=cm, probs_m=pm, aux_m=auxm)
    out = {}
    for mode in ("entropy", "cv", "l2"):
        torch.manual_seed(1)
        rb = ref_single.TopKBalancedRouter(H, E, K, balance_coefficient=0.01, balance_mode=mode)
        with torch.no_grad():
            d, c, p, aux = rb(x)
        out[mode] = dict(weights=sd(rb), probs=p, aux=aux, dispatch=d, combine=c)
    flat = {"x": x}
    for mode, dct in out.items():
        for k, v in dct.items():
            if isinstance(v, dict):
                for kk, vv in v.items():
                    flat[f"{mode}/{k}/{kk}"] = vv
            else:
                flat[f"{mode}/{k}"] = v
    save("router_topk_balanced_single", **flat)

    # R3: core/single PiKVRouter, three consecutive calls (state carries over),
    # cache_update_interval=2 so the correction factor is refreshed inside the run
    torch.manual_seed(2)
    pr = ref_single.PiKVRouter(H, E, K, cache_update_interval=2)
    kv = torch.randn(2, 16, H)
    w0 = sd(pr)
    calls = {}
    with torch.no_grad():
        for i in range(3):
            xi = torch.randn(2, 16, H)
            d, c, p, aux, imp = pr(xi, kv_states=kv if i == 1 else None)
            calls[f"call{i}/x"] = xi
            calls[f"call{i}/dispatch"] = d
            calls[f"call{i}/combine"] = c
            calls[f"call{i}/probs"] = p
            calls[f"call{i}/aux"] = aux
            calls[f"call{i}/importance"] = imp
            calls[f"call{i}/history"] = pr.cache_usage_history.clone()
            calls[f"call{i}/factor"] = pr.cache_correction_factor.detach().clone()
    save("router_pikv_single", kv=kv, weights=w0, **calls)

    # R4: module BaseRouter / TopKBalancedRouter / PiKVRouter (running-count slots)
    torch.manual_seed(3)
    H2, E2 = 32, 4
    x2 = torch.randn(2, 12, H2)
    mb = ref_module.BaseRouter(H2, E2, 2, capacity_factor=1.0)
    with torch.no_grad():
        logits = mb.router(x2)
        d, c, p, aux = mb(x2)
    save("router_base_module", x=x2, logits=logits, weights=sd(mb), dispatch=d, combine=c, probs=p,
         aux=aux, usage=mb.expert_usage_count, total=mb.total_tokens)
    flat = {"x": x2}
    for mode in ("entropy", "variance", "gini"):
        torch.manual_seed(4)
        mt = ref_module.TopKBalancedRouter(H2, E2, 2, balance_mode=mode)
        with torch.no_grad():
            d, c, p, aux = mt(x2)
        for k, v in sd(mt).items():
            flat[f"{mode}/weights/{k}"] = v
        flat[f"{mode}/probs"] = p
        flat[f"{mode}/aux"] = aux
        flat[f"{mode}/dispatch"] = d
        flat[f"{mode}/combine"] = c
    save("router_topk_balanced_module", **flat)
    torch.manual_seed(5)
    mp = ref_module.PiKVRouter(H2, E2, 2)
    mp.update_cache_usage(1, 0.75)
    mp.update_cache_usage(3, 0.25)
    w0 = sd(mp)
    with torch.no_grad():
        d, c, p, aux, imp = mp(x2)
    save("router_pikv_module", x=x2, weights=w0, dispatch=d, combine=c, probs=p, aux=aux, importance=imp,
         usage=mp.expert_usage_count)
    torch.manual_seed(8)
    ma = ref_module.AdaptiveRouter(H2, E2, 2, importance_threshold=0.5)
    w0 = sd(ma)
    with torch.no_grad():
        d, c, p, aux, imp = ma(x2)
    save("router_adaptive_module", x=x2, weights=w0, dispatch=d, combine=c, probs=p, aux=aux, importance=imp,
         usage=ma.expert_usage_count, history=ma.importance_history, history_idx=ma.importance_idx)

    # R5: routing_strategy.AdaptiveRouter (the router PiKVMoE wires up)
    torch.manual_seed(6)
    ar = ref_strategy.AdaptiveRouter(H, E, top_k=2)
    with torch.no_grad():
        rw, idx, tw, lb, imp = ar(x)
        lb_w, lb_i, lb_t, lb_l = ar.load_balancing_router(x)
    save("router_strategy_adaptive", x=x, weights=sd(ar), routing_weights=rw, expert_indices=idx,
         top_k_weights=tw, lb_loss=lb, importance=imp, lb_weights=lb_w, lb_indices=lb_i, lb_topk=lb_t,
         lb_loss_inner=lb_l)


def quant_fixtures(ref_single_c, ref_module_c):
    torch.manual_seed(10)
    k = torch.randn(2, 24, 64)
    v = torch.randn(2, 24, 64) * 3.0 + 0.5
    k[..., 5] *= 20.0
    out = {"keys": k, "values": v}
    # Q1: core/single asymmetric, "8-bit per-channel" (group_size=1) and 4-bit g=16
    for tag, bits, g in (("b8g1", 8, 1), ("b4g16", 4, 16), ("b8g64", 8, 64)):
        qc = ref_single_c.QuantizedCompressor(64, bits=bits, group_size=g)
        with torch.no_grad():
            dk, dv = qc(k, v)
        out[f"single_{tag}/dq_keys"] = dk
        out[f"single_{tag}/dq_values"] = dv
        out[f"single_{tag}/quantization_error"] = qc.quantization_error
        out[f"single_{tag}/sample_count"] = qc.sample_count
    # static (calibrate once) mode: the first group of the keys fixes scale and zero point
    qs = ref_single_c.QuantizedCompressor(64, bits=8, group_size=16, dynamic_quantization=False)
    with torch.no_grad():
        dk, dv = qs(k, v)
    out["single_static/dq_keys"] = dk
    out["single_static/dq_values"] = dv
    out["single_static/scale"] = qs.scale
    out["single_static/zero_point"] = qs.zero_point
    # Q2: module variant, symmetric and asymmetric
    for tag, bits, g, sym in (("b8g32s", 8, 32, True), ("b4g32a", 4, 32, False), ("b4g16s", 4, 16, True),
                              ("b8g64a", 8, 64, False)):
        qc = ref_module_c.QuantizedCompressor(64, bits=bits, group_size=g, symmetric=sym)
        with torch.no_grad():
            dk, dv = qc(k, v)
        out[f"module_{tag}/dq_keys"] = dk
        out[f"module_{tag}/dq_values"] = dv
        out[f"module_{tag}/quantization_error"] = qc.quantization_error
    save("quant_block", **out)

    # per-slice: _quantize_tensor on [1, group] slices (the streaming cache's granularity)
    torch.manual_seed(11)
    H, G = 256, 128
    x = torch.randn(12, H)
    x[:, 7] *= 20.0
    x[3] = 0.0                      # all-equal slice: exercises x_max = x_min + 1e-5
    x[4, :128] = 2.5                # constant non-zero slice
    x[5, 128:] = x[5, 128:].abs() + 100.0   # large offset: big zero point in the asymmetric case
    x = x.bfloat16().float()        # bf16-representable, as the cache input is bf16
    out = {"x": x}
    for tag, bits, sym in (("int8_sym", 8, True), ("int4_asym", 4, False), ("int8_asym", 8, False),
                           ("int4_sym", 4, True)):
        qc = ref_module_c.QuantizedCompressor(H, bits=bits, group_size=G, symmetric=sym)
        q = torch.zeros_like(x)
        dq = torch.zeros_like(x)
        sc = torch.zeros(x.shape[0], H // G)
        with torch.no_grad():
            for t in range(x.shape[0]):
                for g in range(H // G):
                    qq, dd, s = qc._quantize_tensor(x[t:t + 1, g * G:(g + 1) * G])
                    q[t, g * G:(g + 1) * G] = qq
                    dq[t, g * G:(g + 1) * G] = dd
                    sc[t, g] = s
        out[f"{tag}/q"] = q
        out[f"{tag}/dq"] = dq
        out[f"{tag}/scale"] = sc
    save("quant_slices", **out)


def h2o_fixtures(ref_sched):
    torch.manual_seed(20)
    n, hid = 200, 16
    sch = ref_sched.H2OScheduler(256, hid, heavy_ratio=0.1, recent_ratio=0.05)
    out = {}
    # H2OScheduler.update_attention_scores (cache_scheduling.py:69-73) raises under
    # torch >= 2.1 ("Index put requires the source and destination dtypes match":
    # it stores the int64 current_time into the float timestamp buffer), so the
    # accumulate step cannot be run; record that and fill the buffers directly with
    # tie-free values, for which torch.topk is unambiguous.
    try:
        sch.update_attention_scores(torch.arange(4), torch.ones(4))
        out["update_raises"] = np.int64(0)
        sch.attention_accumulator.zero_()
        sch.access_timestamps.zero_()
    except RuntimeError:
        out["update_raises"] = np.int64(1)
        sch.attention_accumulator.zero_()
    sch.attention_accumulator[:n] = torch.rand(n) * 5 + torch.arange(n) * 1e-3
    sch.access_timestamps[:n] = torch.randperm(n).float()
    keys = torch.randn(n, hid)
    mask = sch.select_eviction_candidates(keys, keys, {})
    out["acc"] = sch.attention_accumulator.clone()
    out["ts"] = sch.access_timestamps.clone()
    out["evict_mask"] = mask
    out["n"] = np.int64(n)
    save("h2o_select", **out)

    # manager: evict-then-append sequence (cache 64 x 8, five updates of [2,10,8])
    torch.manual_seed(21)
    mgr = ref_sched.CacheSchedulingManager(64, 8, ref_sched.SchedulingPolicy.H2O)
    out = {}
    for step in range(5):
        kk = torch.randn(2, 10, 8)
        vv = torch.randn(2, 10, 8)
        # give the scheduler tie-free scores over the rows that are currently valid
        cur = int(mgr.cache_size_current.item())
        if cur > 0:
            mgr.scheduler.attention_accumulator[:cur] = torch.rand(cur) + torch.arange(cur) * 1e-3
            mgr.scheduler.access_timestamps[:cur] = torch.randperm(cur).float()
        out[f"s{step}/acc"] = mgr.scheduler.attention_accumulator.clone()
        out[f"s{step}/ts"] = mgr.scheduler.access_timestamps.clone()
        mgr.update_cache(kk, vv)
        out[f"s{step}/keys_in"] = kk
        out[f"s{step}/values_in"] = vv
        out[f"s{step}/cache_keys"] = mgr.cache_keys.clone()
        out[f"s{step}/cache_values"] = mgr.cache_values.clone()
        out[f"s{step}/size"] = mgr.cache_size_current.clone()
        out[f"s{step}/evictions"] = mgr.scheduler.eviction_count.clone()
    save("h2o_manager", **out)


def policy_fixtures(ref_sched):
    """The other eviction policies, called directly with more rows than cache_size (through the manager they
    never see that): buffers hold cache_size scores, so only the first cache_size rows can be chosen."""
    torch.manual_seed(77)
    C, H, n = 48, 8, 64
    keys = torch.randn(n, H)
    out = {"keys": keys}

    def tie_free(scale=1.0):
        return (torch.randperm(C).float() + torch.rand(C) * 0.5) * scale

    st = ref_sched.StreamingLLMScheduler(C, H, start_size=4, recent_size=20)
    out["streaming/mask"] = st.select_eviction_candidates(keys, keys, {})
    out["streaming/small"] = st.select_eviction_candidates(keys[:40], keys[:40], {})
    lru = ref_sched.LRUScheduler(C, H)
    lru.access_times.copy_(tie_free())
    out["lru/access_times"] = lru.access_times
    out["lru/mask"] = lru.select_eviction_candidates(keys, keys, {})
    lp = ref_sched.LRUPlusScheduler(C, H)
    lp.access_times.copy_(tie_free())
    lp.access_frequency.copy_(tie_free())
    lp.importance_scores.copy_(torch.rand(C))
    for k in ("access_times", "access_frequency", "importance_scores"):
        out[f"lru_plus/{k}"] = getattr(lp, k)
    out["lru_plus/priority"] = lp.compute_priority_scores(n)
    out["lru_plus/mask"] = lp.select_eviction_candidates(keys, keys, {})
    fg = ref_sched.FlexGenScheduler(C, H)
    fg.access_frequency.copy_(tie_free())
    fg.access_cost.copy_(torch.rand(C) + 0.5)
    out["flexgen/access_frequency"], out["flexgen/access_cost"] = fg.access_frequency, fg.access_cost
    out["flexgen/mask"] = fg.select_eviction_candidates(keys, keys, {})
    for tag, thr in (("few", 0.001), ("many", 5.0)):        # under the threshold: too few / enough
        q = ref_sched.QUESTScheduler(C, H, quality_threshold=thr)
        q.quality_scores.copy_(torch.rand(C) * 0.9 + 0.1)
        q.usage_frequency.copy_(tie_free(0.25) + 1.0)
        q.last_access_time.copy_(torch.randperm(C).float())
        q.global_time.fill_(C)
        for k in ("quality_scores", "usage_frequency", "last_access_time"):
            out[f"quest_{tag}/{k}"] = getattr(q, k)
        out[f"quest_{tag}/utility"] = q.compute_utility_scores(n)
        out[f"quest_{tag}/mask"] = q.select_eviction_candidates(keys, keys, {})
    # the update methods (whether they run at all under this torch is part of the record)
    for name, fn in (("lru", lambda: ref_sched.LRUScheduler(C, H).update_access_time(torch.tensor([1, 2]))),
                     ("flexgen", lambda: ref_sched.FlexGenScheduler(C, H).update_access_patterns(torch.tensor([1, 2]), torch.tensor([2.0, 3.0])))):
        try:
            fn()
            out[f"{name}/update_raises"] = np.array(0)
        except Exception:
            out[f"{name}/update_raises"] = np.array(1)
    # through the manager these policies never evict: the cache fills up and stops
    mgr = ref_sched.CacheSchedulingManager(16, H, ref_sched.SchedulingPolicy.LRU)
    for i in range(3):
        mgr.update_cache(keys[None, 7 * i: 7 * i + 7], keys[None, 7 * i: 7 * i + 7])
    out["manager_lru/keys"], out["manager_lru/size"] = mgr.cache_keys, mgr.cache_size_current
    save("eviction_policies", **out)


def module_policy_fixtures(ref_msched):
    """AdaKV and DuoAttention of core/single/module/pikv_scheduling.py, called with more rows than cache_size."""
    torch.manual_seed(78)
    C, H, n = 48, 8, 64
    keys = torch.randn(n, H)
    out = {"keys": keys}
    ada = ref_msched.AdaKVScheduler(C, H, compression_ratio=0.5, safeguard_ratio=0.2)
    with torch.no_grad():
        ada.update_importance(torch.arange(C), keys[:C])
    out["adakv/weights/weight"], out["adakv/weights/bias"] = ada.linear_proj.weight, ada.linear_proj.bias
    out["adakv/importance_scores"] = ada.importance_scores
    out["adakv/mask"] = ada.select_eviction_candidates(keys, keys, {})
    out["adakv/small"] = ada.select_eviction_candidates(keys[:40], keys[:40], {})
    duo = ref_msched.DuoAttentionScheduler(C, H, sink_size=5, recent_size=17)
    out["duo/mask"] = duo.select_eviction_candidates(keys, keys, {})
    out["duo/small"] = duo.select_eviction_candidates(keys[:40], keys[:40], {})
    out["duo/evictions"] = duo.eviction_count.clone()
    save("eviction_policies_module", **out)


def attention_fixture(ref_attn):
    torch.manual_seed(30)
    att = ref_attn.PiKVAttention(hidden_size=64, num_heads=4, dropout=0.0)
    att.eval()
    q = torch.randn(3, 1, 4, 16)
    k = torch.randn(3, 40, 4, 16)
    v = torch.randn(3, 40, 4, 16)
    with torch.no_grad():
        ctx = att._compute_attention(q, k, v)
    save("attention_decode", q=q, k=k, v=v, context=ctx)


def rope_fixture(ref_attn):
    """RotaryEmbedding of core/single/pikv_attention.py on head dim 128: tables and rotated q / k."""
    torch.manual_seed(31)
    rope = ref_attn.RotaryEmbedding(128, max_position_embeddings=96)
    q = torch.randn(2, 24, 3, 128)
    k = torch.randn(2, 24, 3, 128).bfloat16().float()          # bf16-valued keys, as the cache path feeds them
    pos = torch.stack([torch.arange(24), torch.randperm(96)[:24]])
    q_out, k_out = rope(q, k, pos)
    save("rope", q=q, k=k, positions=pos, cos=rope.cos_cached, sin=rope.sin_cached, q_out=q_out, k_out=k_out)


def lowrank_fixtures(ref_single_c, ref_module_c, ref_cachec):
    torch.manual_seed(40)
    H = 64
    k = torch.randn(2, 10, H)
    v = torch.randn(2, 10, H)
    svd = ref_single_c.SVDCompressor(H, rank=16)
    with torch.no_grad():
        rk, rv = svd(k, v)
    save("lowrank_svd_single", keys=k, values=v, weights=sd(svd), rec_keys=rk, rec_values=rv)
    torch.manual_seed(41)
    svdm = ref_module_c.SVDCompressor(H, rank=16, adaptive_rank=True, energy_threshold=0.5)
    with torch.no_grad():
        rk, rv = svdm(k, v)
    save("lowrank_svd_module", keys=k, values=v, weights=sd(svdm), rec_keys=rk, rec_values=rv,
         effective_rank=svdm.effective_rank)
    torch.manual_seed(42)
    pyr = ref_single_c.PyramidCompressor(H, compression_ratio=0.5, num_levels=3, decay_factor=0.8)
    imp = torch.rand(2, 10) + torch.arange(20).reshape(2, 10) * 1e-3
    with torch.no_grad():
        uk, uv = pyr(k, v)
        ik, iv = pyr(k, v, imp)
    save("pyramid_single", keys=k, values=v, importance=imp, weights=sd(pyr), uni_keys=uk, uni_values=uv,
         imp_keys=ik, imp_values=iv)
    torch.manual_seed(43)
    cc = ref_cachec.KVCacheCompressor(H, compression_type="pyramid", compression_ratio=0.5)
    with torch.no_grad():
        ck, cv = cc(k, v, imp)
        nk, nv = cc(k, v)
    torch.manual_seed(14)
    pm = ref_module_c.PyramidCompressor(64, compression_ratio=0.5, num_levels=3)
    impm = torch.rand(2, 10)
    wpm = sd(pm)
    with torch.no_grad():
        mk, mv = pm(k, v, impm)
        nk2, nv2 = pm(k, v)
    save("pyramid_module", keys=k, values=v, importance=impm, weights=wpm, ck=mk, cv=mv, nk=nk2, nv=nv2,
         levels=pm._assign_compression_levels(impm), stats=np.array([float(pm.total_compressed_size)]))
    save("cache_pyramid", keys=k, values=v, importance=imp, weights=sd(cc), ck=ck, cv=cv, nk=nk, nv=nv)


def moe_fixture(reference):
    """PiKVMoE (config 1: [8,128,256] fp32, 4 experts, top-2, caches 128..88) built after manual_seed(0),
    two forwards, plain ring caches and H2O-scheduled caches.  Only slices of the [8,128,50257] logits
    are kept.  core/single/distillation.py:9 imports itself, so the module is loaded with that line left
    out (in memory; the reference tree is not touched)."""
    import types
    import core.single  # noqa: F401
    path = os.path.join(reference, "core", "single", "distillation.py")
    lines = open(path).read().split("\n")
    mod = types.ModuleType("core.single.distillation")
    mod.__package__, mod.__file__ = "core.single", path
    sys.modules["core.single.distillation"] = mod
    exec(compile("\n".join(l for i, l in enumerate(lines) if i != 8), path, "exec"), mod.__dict__)
    from core.single.pikv_moe import PiKVMoE
    from core.single.cache_scheduling import SchedulingPolicy
    out = {}
    for tag, kw in (("plain", {}), ("h2o", dict(use_cache_scheduling=True, cache_scheduling_policy=SchedulingPolicy.H2O))):
        torch.manual_seed(0)
        m = PiKVMoE(**kw)
        m.eval()
        g = torch.Generator().manual_seed(1)
        with torch.no_grad():
            for step in range(2):
                x = torch.randn(8, 128, 256, generator=g)
                logits = m(x)
                out[f"{tag}/logits_head{step}"] = logits[:, :, :48].numpy().copy()
                out[f"{tag}/logits_stride{step}"] = logits[:, ::16, ::997].numpy().copy()
                out[f"{tag}/logits_absmax{step}"] = np.float32(logits.abs().max())
        out[f"{tag}/cache_ptrs"] = m.cache_ptrs.numpy().copy()
        out[f"{tag}/n_params"] = np.int64(sum(p.numel() for p in m.parameters()))
        out[f"{tag}/param_sum"] = np.float64(sum(p.double().sum().item() for p in m.parameters()))
    save("pikv_moe_c1", **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference (NoakLiu/PiKV)")
    ap.add_argument("--only", default=None, help="write just this fixture")
    args = ap.parse_args()
    global ONLY
    ONLY = args.only
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    torch.set_num_threads(1)
    from core.single import pikv_routing, pikv_compression, cache_scheduling, routing_strategy
    from core.single import kv_cache_compression, pikv_attention
    from core.single.module import pikv_routing as m_routing, pikv_compression as m_compression

    router_fixtures(pikv_routing, m_routing, routing_strategy)
    quant_fixtures(pikv_compression, m_compression)
    h2o_fixtures(cache_scheduling)
    policy_fixtures(cache_scheduling)
    from core.single.module import pikv_scheduling as m_scheduling
    module_policy_fixtures(m_scheduling)
    attention_fixture(pikv_attention)
    rope_fixture(pikv_attention)
    lowrank_fixtures(pikv_compression, m_compression, kv_cache_compression)
    torch.set_num_threads(4)
    moe_fixture(args.reference)


if __name__ == "__main__":
    main()
