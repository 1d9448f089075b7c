"""CPU oracle for the routed KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain numpy (fp32 IEEE arithmetic, round-half-even),
the arithmetic of the reference's PyTorch operators for the routed KV-cache
path.  It exists so that the CUDA kernels can be checked on a machine that
does not have the reference checked out.  Only the test-suite, the smoke test
and the benchmark's CPU-baseline leg may import it; the product package never
does and fails loudly when its CUDA library is missing.

Pinning: every function here is checked against outputs of the reference's
own modules on seeded inputs (fixtures under tests/golden/, produced by
tests/golden/make_golden.py, which imports the reference).  The reference has
no assertions or golden vectors of its own for this path.

Citations are paths inside the reference project.
"""
from __future__ import annotations

import math
import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even) and return it as fp32."""
    x = np.ascontiguousarray(x, dtype=F32)
    u = x.view(np.uint32).astype(np.uint64)
    rounding = ((u >> 16) & 1) + 0x7FFF
    u = ((u + rounding) >> 16) << 16
    out = (u & 0xFFFFFFFF).astype(np.uint32).view(F32)
    nan = np.isnan(x)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out.reshape(x.shape)


def stable_topk(values: np.ndarray, k: int):
    """Top-k along the last axis, descending, ties broken by LOWEST index.

    The reference calls torch.topk (core/single/pikv_routing.py:76,
    core/single/cache_scheduling.py:87,90), whose tie order is unspecified;
    this is the same selection with a stable descending sort.
    """
    v = np.asarray(values)
    order = np.argsort(-v, axis=-1, kind="stable")
    # argsort of -v is stable ascending on -v == descending on v, lowest index first
    idx = order[..., :k]
    return np.take_along_axis(v, idx, axis=-1), idx.astype(np.int64)


def softmax_f32(x: np.ndarray) -> np.ndarray:
    """softmax over the last axis in fp32 (F.softmax, pikv_routing.py:73)."""
    x = np.asarray(x, dtype=F32)
    m = x.max(axis=-1, keepdims=True)
    e = np.exp((x - m).astype(F32)).astype(F32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)


# --------------------------------------------------------------------------
# R - router gate
# --------------------------------------------------------------------------
def gate_logits(a: np.ndarray, w2: np.ndarray, b2: np.ndarray | None) -> np.ndarray:
    """Last layer of the gate net: a @ w2.T + b2 in fp32.

    core/single/pikv_routing.py:34-38,65 (nn.Linear(hidden, num_experts)).
    `a` is the post-ReLU activation of the first layer.
    """
    out = np.asarray(a, F32) @ np.asarray(w2, F32).T
    if b2 is not None:
        out = out + np.asarray(b2, F32)
    return out.astype(F32)


def gate_tail(logits: np.ndarray, top_k: int, *, expert_mask=None, correction=None,
              temperature: float = 1.0, mask_mode: str = "single", renorm_eps: float = 0.0):
    """logits -> (probs, topk_idx, topk_w).

    Order of operations follows PiKVRouter.forward
    (core/single/pikv_routing.py:457-473): multiply by the cache correction
    factor, add the availability mask, softmax, top-k of the probabilities,
    renormalise.  ExpertRouter divides by a temperature first and treats the
    mask as an additive bias (core/single/routing_strategy.py:42-53).

    mask_mode: "single"  logits + (1-mask) * -1e9        (pikv_routing.py:70)
               "module"  logits + (1-mask) * finfo.min   (module/pikv_routing.py:133-134)
               "bias"    logits + mask                   (routing_strategy.py:46)
    renorm_eps: 0 for core/single (pikv_routing.py:79), 1e-8 for the module
                variant (module/pikv_routing.py:143).
    """
    l = np.asarray(logits, dtype=F32)
    if temperature != 1.0:
        l = (l / F32(temperature)).astype(F32)
    if correction is not None:
        l = (l * np.asarray(correction, F32)).astype(F32)
    if expert_mask is not None:
        m = np.asarray(expert_mask, F32)
        if mask_mode == "single":
            l = (l + ((F32(1) - m) * F32(-1e9)).astype(F32)).astype(F32)
        elif mask_mode == "module":
            l = (l + ((F32(1) - m) * np.finfo(F32).min).astype(F32)).astype(F32)
        elif mask_mode == "bias":
            l = (l + m).astype(F32)
        else:
            raise ValueError(mask_mode)
    probs = softmax_f32(l)
    top_p, top_i = stable_topk(probs, top_k)
    denom = top_p.sum(axis=-1, keepdims=True, dtype=F32)
    if renorm_eps:
        denom = (denom + F32(renorm_eps)).astype(F32)
    top_w = (top_p / denom).astype(F32)
    return probs, top_i, top_w


def topk_margin(probs: np.ndarray, top_k: int) -> np.ndarray:
    """Relative gap between the k-th and (k+1)-th probability of each token.

    Used by the parity tests to tell a real index mismatch from a near-tie
    flipped by a different fp32 accumulation order of the gate GEMM.
    """
    s = -np.sort(-np.asarray(probs, F32), axis=-1)
    if s.shape[-1] <= top_k:
        return np.full(s.shape[:-1], np.inf, F32)
    a, b = s[..., top_k - 1], s[..., top_k]
    return (a - b) / np.maximum(a, F32(1e-30))


def capacity(num_tokens: int, capacity_factor: float, top_k: int, num_experts: int) -> int:
    """core/single/pikv_routing.py:40-42 (same in module/pikv_routing.py:62-65)."""
    return int(num_tokens * capacity_factor * top_k / num_experts)


def slot_assign(topk_idx: np.ndarray, num_experts: int, cap: int):
    """Running per-expert position in (token, k) order; -1 once an expert is full.

    core/single/module/pikv_routing.py:88-104.  Returns (slot[T,k] int32,
    counts_k[k,E] int32) where counts_k counts every selection, dropped or not
    (that is what expert_usage_count accumulates, module/pikv_routing.py:157-160).
    """
    idx = np.asarray(topk_idx).reshape(-1, topk_idx.shape[-1])
    T, K = idx.shape
    used = np.zeros(num_experts, np.int64)
    slot = np.full((T, K), -1, np.int32)
    for t in range(T):
        for k in range(K):
            e = idx[t, k]
            if used[e] < cap:
                slot[t, k] = used[e]
                used[e] += 1
    counts_k = np.zeros((K, num_experts), np.int32)
    for k in range(K):
        counts_k[k] = np.bincount(idx[:, k], minlength=num_experts)
    return slot, counts_k


def slot_assign_fast(topk_idx: np.ndarray, num_experts: int, cap: int):
    """Vectorised slot_assign for large T (same result, no Python loop)."""
    idx = np.asarray(topk_idx).reshape(-1, topk_idx.shape[-1])
    T, K = idx.shape
    flat = idx.reshape(-1)
    onehot = np.zeros((flat.size, num_experts), np.int32)
    onehot[np.arange(flat.size), flat] = 1
    excl = np.cumsum(onehot, axis=0) - onehot
    pos = excl[np.arange(flat.size), flat].astype(np.int32)
    slot = np.where(pos < cap, pos, -1).astype(np.int32).reshape(T, K)
    counts_k = np.stack([np.bincount(idx[:, k], minlength=num_experts) for k in range(K)]).astype(np.int32)
    return slot, counts_k


def dispatch_combine_module(topk_idx, topk_w, num_experts: int, cap: int):
    """Dense [T,E,cap] dispatch/combine, running-count positions.

    core/single/module/pikv_routing.py:67-106.
    """
    slot, _ = slot_assign(topk_idx, num_experts, cap)
    T, K = slot.shape
    d = np.zeros((T, num_experts, cap), F32)
    c = np.zeros((T, num_experts, cap), F32)
    for t in range(T):
        for k in range(K):
            if slot[t, k] >= 0:
                d[t, topk_idx[t, k], slot[t, k]] = 1.0
                c[t, topk_idx[t, k], slot[t, k]] = topk_w[t, k]
    return d, c


def dispatch_combine_single(topk_idx, topk_w, num_experts: int, cap: int):
    """Dense [T,E,cap] dispatch/combine exactly as core/single builds them.

    core/single/pikv_routing.py:101-128.  `expert_count[idx] += 1` with repeated
    indices is a non-accumulating index_put and the positions are read before the
    update, so in pass i every token routed to expert e lands in the position
    "number of earlier passes in which e was chosen by any token".
    """
    idx = np.asarray(topk_idx)
    T, K = idx.shape
    d = np.zeros((T, num_experts, cap), F32)
    c = np.zeros((T, num_experts, cap), F32)
    count = np.zeros(num_experts, np.int64)
    for i in range(K):
        e = idx[:, i]
        ok = count[e] < cap
        pos = count[e[ok]]
        t_ok = np.nonzero(ok)[0]
        d[t_ok, e[ok], pos] = 1.0
        c[t_ok, e[ok], pos] = np.asarray(topk_w, F32)[t_ok, i]
        count[np.unique(e[ok])] += 1
    return d, c


def aux_loss_base(probs: np.ndarray, num_experts: int) -> np.float32:
    """sum(p_bar * log(p_bar * E + 1e-9)), core/single/pikv_routing.py:155-159."""
    p = np.asarray(probs, F32).reshape(-1, num_experts).mean(axis=0, dtype=F32)
    return F32(np.sum(p * np.log(p * F32(num_experts) + F32(1e-9)), dtype=F32))


def aux_loss_topk_balanced(probs, num_experts: int, coef: float, mode: str) -> np.float32:
    """TopKBalancedRouter extra term, core/single/pikv_routing.py:194-220."""
    p = np.asarray(probs, F32).reshape(-1, num_experts).mean(axis=0, dtype=F32)
    base = aux_loss_base(probs, num_experts)
    if mode == "entropy":
        term = -np.sum(p * np.log(p + F32(1e-9)), dtype=F32) / F32(math.log(num_experts))
        bal = F32(-coef) * term
    elif mode == "cv":
        mean = p.mean(dtype=F32)
        std = p.std(ddof=1, dtype=F32)
        bal = F32(coef) * (std / (mean + F32(1e-9)))
    else:
        uni = F32(1.0) / F32(num_experts)
        bal = F32(coef) * np.sum((p - uni) ** 2, dtype=F32)
    return F32(base + bal)


def aux_loss_module(probs, topk_idx, num_experts: int) -> np.float32:
    """E * sum_e p_bar_e * f_e, core/single/module/pikv_routing.py:164-181."""
    p = np.asarray(probs, F32).reshape(-1, num_experts).mean(axis=0, dtype=F32)
    idx = np.asarray(topk_idx).reshape(-1)
    f = (np.bincount(idx, minlength=num_experts) / F32(idx.size)).astype(F32)
    return F32(np.sum(p * f, dtype=F32) * F32(num_experts))


# --------------------------------------------------------------------------
# Q - quantisation
# --------------------------------------------------------------------------
def qrange(bits: int, symmetric: bool):
    """core/single/module/pikv_compression.py:947-963; asymmetric branch equals
    core/single/pikv_compression.py:400-405."""
    if symmetric and bits in (4, 8, 16):
        return -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    return 0, (1 << bits) - 1


def quantize_block(x: np.ndarray, bits: int, symmetric: bool):
    """Quantise ONE block with block-wide statistics.

    core/single/module/pikv_compression.py:965-1006 (`_quantize_tensor`, dynamic
    branch); with symmetric=False this is also core/single/pikv_compression.py:
    408-422 (`_quantize`).  Returns (q, dq, scale, zero_point), all fp32.
    """
    x = np.asarray(x, F32)
    qmin, qmax = qrange(bits, symmetric)
    x_min = F32(x.min())
    x_max = F32(x.max())
    if x_max == x_min:
        x_max = F32(x_min + F32(1e-5))
    if symmetric:
        abs_max = max(abs(x_min), abs(x_max))
        scale = F32(F32(2) * abs_max) / F32(qmax - qmin)
        zp = F32(0.0)
    else:
        scale = F32(x_max - x_min) / F32(qmax - qmin)
        zp = F32(qmin) - F32(np.rint(F32(x_min / scale)))
    scale = F32(scale)
    zp = F32(zp)
    q = np.clip(np.rint((x / scale).astype(F32) + zp).astype(F32), qmin, qmax).astype(F32)
    dq = ((q - zp).astype(F32) * scale).astype(F32)
    return q, dq, scale, zp


def quant_block_forward(x2d: np.ndarray, bits: int, group_size: int, symmetric: bool):
    """QuantizedCompressor.forward on one tensor: every column group of width
    `group_size` is one block with statistics over ALL rows.

    core/single/pikv_compression.py:483-500, module/pikv_compression.py:1031-1037.
    Returns (dq[N,H], q[N,H], scale[G], zp[G], mse_last_group).
    """
    x2d = np.asarray(x2d, F32)
    N, H = x2d.shape
    dq = np.zeros_like(x2d)
    q = np.zeros_like(x2d)
    scales, zps = [], []
    mse = F32(0)
    for i in range(0, H, group_size):
        end = min(i + group_size, H)
        qq, dd, s, z = quantize_block(x2d[:, i:end], bits, symmetric)
        dq[:, i:end] = dd
        q[:, i:end] = qq
        scales.append(s)
        zps.append(z)
        mse = F32(np.mean((x2d[:, i:end] - dd) ** 2, dtype=F32))
    return dq, q, np.array(scales, F32), np.array(zps, F32), mse


def quant_token_groups(x2d: np.ndarray, bits: int, group_size: int, symmetric: bool):
    """Streaming-cache granularity: `_quantize_tensor` applied to every
    [1, group_size] slice (one token, one group).  Same function as above
    (module/pikv_compression.py:945-1012), slice granularity.

    Returns (q[N,H] fp32 integer-valued, scale[N,G] fp32, zp[N,G] fp32).
    """
    x = np.asarray(x2d, F32)
    N, H = x.shape
    G = H // group_size
    xg = x.reshape(N, G, group_size)
    qmin, qmax = qrange(bits, symmetric)
    x_min = xg.min(axis=-1)
    x_max = xg.max(axis=-1)
    x_max = np.where(x_max == x_min, (x_min + F32(1e-5)).astype(F32), x_max).astype(F32)
    if symmetric:
        abs_max = np.maximum(np.abs(x_min), np.abs(x_max)).astype(F32)
        scale = ((F32(2) * abs_max).astype(F32) / F32(qmax - qmin)).astype(F32)
        zp = np.zeros_like(scale)
    else:
        scale = ((x_max - x_min).astype(F32) / F32(qmax - qmin)).astype(F32)
        zp = (F32(qmin) - np.rint((x_min / scale).astype(F32)).astype(F32)).astype(F32)
    q = np.clip(np.rint(((xg / scale[..., None]).astype(F32) + zp[..., None]).astype(F32)), qmin, qmax)
    return q.reshape(N, H).astype(F32), scale, zp


def dequant_token_groups(q, scale, zp, group_size: int):
    """dq = (q - zp) * scale, module/pikv_compression.py:1006."""
    q = np.asarray(q, F32)
    N, H = q.shape
    G = H // group_size
    qg = q.reshape(N, G, group_size)
    return ((qg - np.asarray(zp, F32)[..., None]).astype(F32) * np.asarray(scale, F32)[..., None]).astype(F32).reshape(N, H)


def routed_append(K, V, topk_idx, slot, num_seqs: int, cap: int, bits: int, symmetric: bool,
                  group_size: int):
    """The composed routed append: for every (token, j) with slot >= 0 store the
    token's quantised K and V rows at [topk_idx[t,j], slot[t,j]].

    Composition of module/pikv_routing.py:93-104 (slot order) with
    module/pikv_compression.py:945-1012 per [1, group] slice.  The reference
    itself does not wire these together (its KVCache stores one mean vector
    per forward, core/single/pikv_moe.py:53-78); the contiguous row copy it
    does perform is core/single/cache_scheduling.py:430-436.

    Returns dict of logical (unpaged) arrays:
      k_codes,v_codes [num_seqs, cap, H] fp32 integer-valued (0 where empty)
      k_scale,v_scale,k_zp,v_zp [num_seqs, cap, G] fp32
      length [num_seqs] int32
    """
    K = np.asarray(K, F32)
    V = np.asarray(V, F32)
    T, H = K.shape
    G = H // group_size
    kq, ks, kz = quant_token_groups(K, bits, group_size, symmetric)
    vq, vs, vz = quant_token_groups(V, bits, group_size, symmetric)
    out = {
        "k_codes": np.zeros((num_seqs, cap, H), F32), "v_codes": np.zeros((num_seqs, cap, H), F32),
        "k_scale": np.zeros((num_seqs, cap, G), F32), "v_scale": np.zeros((num_seqs, cap, G), F32),
        "k_zp": np.zeros((num_seqs, cap, G), F32), "v_zp": np.zeros((num_seqs, cap, G), F32),
        "length": np.zeros(num_seqs, np.int32),
    }
    idx = np.asarray(topk_idx)
    sl = np.asarray(slot)
    t_ix, j_ix = np.nonzero(sl >= 0)
    e = idx[t_ix, j_ix]
    s = sl[t_ix, j_ix]
    out["k_codes"][e, s] = kq[t_ix]
    out["v_codes"][e, s] = vq[t_ix]
    out["k_scale"][e, s] = ks[t_ix]
    out["v_scale"][e, s] = vs[t_ix]
    out["k_zp"][e, s] = kz[t_ix]
    out["v_zp"][e, s] = vz[t_ix]
    np.maximum.at(out["length"], e, (s + 1).astype(np.int32))
    return out


# --------------------------------------------------------------------------
# H - H2O scoring and eviction
# --------------------------------------------------------------------------
def h2o_counts(cache_len: int, heavy_ratio: float, recent_ratio: float):
    """core/single/cache_scheduling.py:83-84."""
    return max(1, int(cache_len * heavy_ratio)), max(1, int(cache_len * recent_ratio))


def h2o_update(acc, ts, current_time: int, indices, weights, decay: float | None = None):
    """core/single/cache_scheduling.py:69-73; decay first in the module variant
    (core/single/module/pikv_scheduling.py:119-125).  In place; returns time+1."""
    if decay is not None:
        acc *= F32(decay)
    acc[indices] = acc[indices] + np.asarray(weights, F32)
    ts[indices] = F32(current_time)
    return current_time + 1


def h2o_select(acc, ts, num_heavy: int, num_recent: int):
    """Eviction mask (True = evict) and ascending kept indices.

    core/single/cache_scheduling.py:86-99 with the stable tie rule, and the
    ascending order of core/single/cache_scheduling.py:418-419.
    """
    acc = np.asarray(acc, F32)
    ts = np.asarray(ts, F32)
    n = acc.shape[0]
    _, heavy = stable_topk(acc, min(num_heavy, n))
    _, recent = stable_topk(ts, min(num_recent, n))
    evict = np.ones(n, bool)
    evict[heavy] = False
    evict[recent] = False
    return evict, np.nonzero(~evict)[0].astype(np.int32)


def manager_update_cache(cache_keys, cache_values, size: int, new_keys, new_values, evict_fn):
    """CacheSchedulingManager.update_cache, core/single/cache_scheduling.py:397-436.

    evict_fn(n) -> bool evict mask over the current n rows.  Returns
    (new_size, evicted_count); cache arrays are modified in place.
    """
    cap = cache_keys.shape[0]
    nk = new_keys.reshape(-1, new_keys.shape[-1])
    nv = new_values.reshape(-1, new_values.shape[-1])
    evicted = 0
    if size + nk.shape[0] > cap:
        evict = evict_fn(size)
        keep = np.nonzero(~evict)[0]
        cache_keys[: len(keep)] = cache_keys[:size][keep]
        cache_values[: len(keep)] = cache_values[:size][keep]
        size = len(keep)
        evicted = int(evict.sum())
    end = min(size + nk.shape[0], cap)
    cache_keys[size:end] = nk[: end - size]
    cache_values[size:end] = nv[: end - size]
    return end, evicted


def token_importance(query, keys, hidden: int):
    """Column sums of softmax(Q K^T / sqrt(hidden)): the accumulated-attention
    score H2O consumes.  core/single/pikv_moe.py:226-247."""
    s = (np.asarray(query, F32) @ np.swapaxes(np.asarray(keys, F32), -1, -2)) / F32(math.sqrt(hidden))
    return softmax_f32(s).sum(axis=-2, dtype=F32)


# --------------------------------------------------------------------------
# A - decode attention on the dequantised cache
# --------------------------------------------------------------------------
def decode_attention(q, k_dq, v_dq, lengths=None):
    """softmax(q K^T / sqrt(d)) V per stream with grouped query heads.

    q [B, Hq, d]; k_dq, v_dq [B, Hkv, ctx, d] (already dequantised with
    module/pikv_compression.py:1006); lengths [B] optional valid context.
    Arithmetic: core/single/pikv_attention.py:117-123,163,188.  Query head h
    reads KV head h // (Hq // Hkv); grouped heads have no counterpart in the
    reference (its heads are 1:1) and reduce to it when Hq == Hkv.
    Returns (out [B,Hq,d] fp32, probs_sum_per_kv [B,Hkv,ctx] fp32) where the
    second output is the sum over the query heads of a group of the attention
    probabilities (the H2O score increment).
    """
    q = np.asarray(q, F32)
    B, Hq, d = q.shape
    Hkv, ctx = k_dq.shape[1], k_dq.shape[2]
    g = Hq // Hkv
    out = np.zeros((B, Hq, d), F32)
    psum = np.zeros((B, Hkv, ctx), F32)
    for b in range(B):
        n = ctx if lengths is None else int(lengths[b])
        for h in range(Hkv):
            kk = np.asarray(k_dq[b, h, :n], F32)
            vv = np.asarray(v_dq[b, h, :n], F32)
            qq = q[b, h * g:(h + 1) * g]
            s = (qq @ kk.T) / F32(math.sqrt(d))
            p = softmax_f32(s)
            out[b, h * g:(h + 1) * g] = p @ vv
            psum[b, h, :n] = p.sum(axis=0, dtype=F32)
    return out, psum


# --------------------------------------------------------------------------
# P - low-rank projection
# --------------------------------------------------------------------------
def lowrank_project(x, w_p, b_p):
    """relu(x @ w_p.T + b_p): the latent the reconstructor consumes.
    core/single/pikv_compression.py:336,341 (F.relu applied to the projection)."""
    y = np.asarray(x, F32) @ np.asarray(w_p, F32).T
    if b_p is not None:
        y = y + np.asarray(b_p, F32)
    return np.maximum(y, 0).astype(F32)


def lowrank_reconstruct(y, w_r, b_r):
    """y @ w_r.T + b_r, core/single/pikv_compression.py:341."""
    out = np.asarray(y, F32) @ np.asarray(w_r, F32).T
    if b_r is not None:
        out = out + np.asarray(b_r, F32)
    return out.astype(F32)


def svd_compress(x, w_p, b_p, w_r, b_r, rank_keep: int | None = None, pad: bool = False):
    """SVDCompressor.forward for one tensor.

    core/single/pikv_compression.py:336-341 truncates the latent to
    `rank_keep` columns and the reconstructor then fails unless rank_keep ==
    rank (the single variant never truncates because its adaptive rank is
    inert); core/single/module/pikv_compression.py:874-885 zero-pads instead
    (pad=True)."""
    z = np.asarray(x, F32) @ np.asarray(w_p, F32).T + np.asarray(b_p, F32)
    if rank_keep is not None and rank_keep < z.shape[-1] and pad:
        z = z.copy()
        z[..., rank_keep:] = 0
    return lowrank_reconstruct(np.maximum(z, 0), w_r, b_r)


def pyramid_uniform(x, enc, dec):
    """PyramidCompressor.forward without importance: relu(enc_i) chain then
    relu(dec_i) chain in reverse.  core/single/pikv_compression.py:202-215.
    enc/dec: lists of (weight, bias)."""
    h = np.asarray(x, F32)
    for w, b in enc:
        h = np.maximum(h @ np.asarray(w, F32).T + np.asarray(b, F32), 0)
    for w, b in reversed(dec):
        h = np.maximum(h @ np.asarray(w, F32).T + np.asarray(b, F32), 0)
    return h.astype(F32)


def pyramid_level_sizes(n: int, num_levels: int, decay: float):
    """core/single/pikv_compression.py:149-160."""
    sizes, remaining = [], n
    for i in range(num_levels):
        if i == num_levels - 1:
            sizes.append(remaining)
        else:
            s = int(remaining * (1 - decay) * (decay ** i))
            sizes.append(s)
            remaining -= s
    return sizes


def pyramid_importance(x2d, importance_flat, enc, dec, num_levels: int, decay: float):
    """PyramidCompressor.forward with importance scores: sort descending, split
    into level buckets, level L applies L encoder layers then L decoder layers.
    core/single/pikv_compression.py:145-196.  The sort must be the same
    permutation the caller's argsort produced; pass tie-free importance."""
    x2d = np.asarray(x2d, F32)
    order = np.argsort(-np.asarray(importance_flat, F32), kind="stable")
    sizes = pyramid_level_sizes(order.size, num_levels, decay)
    out = np.zeros_like(x2d)
    start = 0
    for level, size in enumerate(sizes):
        if size <= 0:
            continue
        ix = order[start:start + size]
        h = x2d[ix]
        for i in range(level):
            h = np.maximum(h @ np.asarray(enc[i][0], F32).T + np.asarray(enc[i][1], F32), 0)
        for i in range(level - 1, -1, -1):
            h = np.maximum(h @ np.asarray(dec[i][0], F32).T + np.asarray(dec[i][1], F32), 0)
        out[ix] = h
        start += size
    return out


def cache_pyramid_compression(x, importance, w1, b1, w2, b2):
    """kv_cache_compression.PyramidCompression: xi = x*imp[...,None];
    xi + L(h/2,h)(L(h,h/2)(xi)).  core/single/kv_cache_compression.py:21-45
    (the residual adds the importance-weighted input, not the raw one)."""
    x = np.asarray(x, F32)
    xi = x if importance is None else (x * np.asarray(importance, F32)[..., None]).astype(F32)
    h = xi @ np.asarray(w1, F32).T + np.asarray(b1, F32)
    h = h @ np.asarray(w2, F32).T + np.asarray(b2, F32)
    return (xi + h).astype(F32)


# --------------------------------------------------------------------------
# D - expert-parallel combine
# --------------------------------------------------------------------------
def module_adaptive_top_k(x, importance, w0, b0, w1, b1, top_k: int) -> int:
    """core/single/module/pikv_routing.py:345-363: k for the whole batch = 1 + argmax of a softmax MLP on
    [mean hidden state, mean importance] (softmax is monotone, so the argmax of the logits)."""
    feats = np.concatenate([x.reshape(-1, x.shape[-1]).mean(0), [importance.mean()]]).astype(F32)
    h = np.maximum(feats @ w0.T + b0, 0)
    return min(int(np.argmax(h @ w1.T + b1)) + 1, top_k)


def module_cache_adjustment(x, hit_rates, w0, b0, w1, b1):
    """core/single/module/pikv_routing.py:453-479: tanh MLP on [mean over the sequence, cache hit rates],
    one row per batch element, broadcast over the sequence."""
    b = x.shape[0]
    inp = np.concatenate([x.mean(1), np.broadcast_to(hit_rates, (b, hit_rates.shape[0]))], axis=1).astype(F32)
    return np.tanh(np.maximum(inp @ w0.T + b0, 0) @ w1.T + b1).astype(F32)


def module_pyramid_levels(importance, thresholds):
    """core/single/module/pikv_compression.py:167-184.  Level 0 doubles as "unassigned" in that loop, so a
    token ends at the first level L >= 1 below the last whose threshold it reaches, else at the last."""
    n = len(thresholds)
    levels = np.full(importance.shape, n - 1, np.int64)
    for level in range(n - 2, 0, -1):
        levels = np.where(importance >= thresholds[level], level, levels)
    return levels


def layer_norm(x, g, b, eps=1e-5):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return ((x - mu) / np.sqrt(var + eps) * g + b).astype(F32)


def module_pyramid(x2d, levels_flat, layers):
    """core/single/module/pikv_compression.py:186-229.  layers[i] = dict(enc_w, enc_b, enc_g, enc_beta, dec_w,
    dec_b, dec_g, dec_beta): a token of level L runs encoders 0..L (Linear, LayerNorm, ReLU), decoders L..0
    (Linear, LayerNorm) and adds the result to itself."""
    out = np.zeros_like(x2d)
    for level in range(len(layers)):
        idx = np.nonzero(levels_flat == level)[0]
        if idx.size == 0:
            continue
        y = x2d[idx]
        for i in range(level + 1):
            L = layers[i]
            y = np.maximum(layer_norm(y @ L["enc_w"].T + L["enc_b"], L["enc_g"], L["enc_beta"]), 0)
        for i in range(level, -1, -1):
            L = layers[i]
            y = layer_norm(y @ L["dec_w"].T + L["dec_b"], L["dec_g"], L["dec_beta"])
        out[idx] = x2d[idx] + y
    return out


def evict_lowest(scores: np.ndarray, num_to_evict: int, cache_len: int) -> np.ndarray:
    """bool [cache_len]: the num_to_evict lowest scores (ties: lowest index first) among the scored entries;
    torch.topk(largest=False) of core/single/cache_scheduling.py:195,245,280,343 with a defined tie order."""
    mask = np.zeros(cache_len, bool)
    order = np.argsort(np.asarray(scores, F32), kind="stable")
    mask[order[:num_to_evict]] = True
    return mask


def streaming_llm_mask(cache_len: int, cache_size: int, start_size: int, recent_size: int) -> np.ndarray:
    """core/single/cache_scheduling.py:114-133."""
    mask = np.zeros(cache_len, bool)
    if cache_len <= cache_size:
        return mask
    mask[start_size:max(start_size, cache_len - recent_size)] = True
    return mask


def lru_plus_priority(access_times, access_frequency, importance, frequency_weight=0.3, importance_weight=0.4):
    """core/single/cache_scheduling.py:311-327."""
    t, f = np.asarray(access_times, F32), np.asarray(access_frequency, F32)
    rec = F32(1.0 - frequency_weight - importance_weight)
    return (rec * (t / (t.max() + F32(1e-8))) + F32(frequency_weight) * (f / (f.max() + F32(1e-8))) +
            F32(importance_weight) * np.asarray(importance, F32)).astype(F32)


def quest_utility(quality, frequency, last_access, global_time: int, decay: float = 0.95):
    """core/single/cache_scheduling.py:164-176."""
    age = (F32(global_time) - np.asarray(last_access, F32)).astype(F32)
    return (np.asarray(quality, F32) * np.asarray(frequency, F32) * np.power(F32(decay), age).astype(F32)).astype(F32)


def quest_mask(utility, threshold: float, cache_len: int, cache_size: int) -> np.ndarray:
    """core/single/cache_scheduling.py:178-203: everything under the threshold (a mask as long as the scored
    entries), or the lowest num_to_evict when those are too few."""
    below = np.asarray(utility, F32) < F32(threshold)
    n_ev = cache_len - cache_size
    return evict_lowest(utility, n_ev, cache_len) if below.sum() < n_ev else below


def adakv_mask(scores: np.ndarray, cache_len: int, cache_size: int, compression_ratio: float) -> np.ndarray:
    """AdaKVScheduler.select_eviction_candidates, core/single/module/pikv_scheduling.py:644-666: keep the
    int(cache_len * (1 - ratio)) highest scores (safeguarded head first, then the rest: one top-k), lowest
    index first among equals; rows without a score (past len(scores)) are evicted."""
    mask = np.zeros(cache_len, bool)
    if cache_len <= cache_size:
        return mask
    mask[:] = True
    keep = int(cache_len * (1 - compression_ratio))
    order = np.argsort(-np.asarray(scores[:cache_len], F32), kind="stable")[:keep]
    mask[order] = False
    return mask


def duo_attention_mask(cache_len: int, cache_size: int, sink_size: int, recent_size: int) -> np.ndarray:
    """DuoAttentionScheduler.select_eviction_candidates, core/single/module/pikv_scheduling.py:687-701."""
    mask = np.zeros(cache_len, bool)
    if cache_len <= cache_size:
        return mask
    mask[:] = True
    mask[:sink_size] = False
    mask[-recent_size:] = False
    return mask


def shard_slot_base(counts_all: np.ndarray, rank: int, lengths: np.ndarray, cap: int):
    """Expert-sharded append, one step: counts_all [world, E] are every rank's selection counts.  Rows of a
    sequence are ordered by source rank, so this rank's first row of sequence e lands at
    lengths[e] + sum of the lower ranks' counts; the sequence grows by the total, cut at the capacity.
    (Placement rule of core/single/cache_scheduling.py:430-436 per destination sequence, exchange of
    core/distributed/distributed_pikv.py:174-194.)  Returns (slot_base [E], new_lengths [E])."""
    counts_all = np.asarray(counts_all, np.int64)
    base = np.asarray(lengths, np.int64) + counts_all[:rank].sum(0)
    new_len = np.asarray(lengths, np.int64) + counts_all.sum(0)
    if cap > 0:
        new_len = np.minimum(new_len, cap)
    return base, new_len


def scale_push_runs(slot_base: np.ndarray, counts: np.ndarray, cap: int, owner_of, rank: int, page_tokens: int = 16):
    """The (sequence, page, first row, end row) runs of scales this rank ships to other GPUs after a sharded
    append: its rows of sequence e are the slots [slot_base[e], slot_base[e] + counts[e]) cut at the
    capacity; sequences it owns itself are skipped."""
    runs = []
    for e in range(len(counts)):
        if owner_of(e) == rank:
            continue
        a = int(slot_base[e])
        b = a + int(counts[e])
        if cap > 0:
            b = min(b, cap)
        for p in range(a // page_tokens, (b - 1) // page_tokens + 1 if b > a else 0):
            runs.append((e, p, max(a - p * page_tokens, 0), min(b - p * page_tokens, page_tokens)))
    return runs


def expert_parallel_combine(expert_outputs, routing_probs, world_size: int):
    """sum over ranks of sum over local experts of out_e * p[..., e].

    core/distributed/distributed_pikv.py:174-194 (contiguous expert split,
    all_reduce SUM).  expert_outputs [E, T, H]; routing_probs [T, E].
    Returns (combined [T,H], per_rank_partials [world, T, H])."""
    E = expert_outputs.shape[0]
    per = E // world_size
    parts = []
    for r in range(world_size):
        acc = np.zeros(expert_outputs.shape[1:], F32)
        for e in range(r * per, (r + 1) * per):
            acc += np.asarray(expert_outputs[e], F32) * np.asarray(routing_probs, F32)[:, e:e + 1]
        parts.append(acc)
    parts = np.stack(parts)
    return parts.sum(axis=0, dtype=F32), parts


def striped_owner(perm, e: int, s: int, pos, stripe: int, world: int):
    """Rank and local slot of row `pos` of the cache of pair (expert e, stream s) when stripes of `stripe`
    tokens rotate over the ranks starting at (perm[e] + s) mod world.  This placement has no counterpart in
    the reference (contiguous expert blocks, core/distributed/distributed_pikv.py:91-96); restated here so
    that the kernels' arithmetic is checked against an independent statement."""
    pos = np.asarray(pos, np.int64)
    c = pos // stripe
    owner = (int(perm[e]) + s + c) % world
    local = (c // world) * stripe + pos % stripe
    return owner, local


def routed_decode_combine(q, k_dq, v_dq, lengths, topk_idx, topk_w, lse_merge: bool = False):
    """Decode output of every stream over the caches of its top-k experts.

    q [S, Hq, d]; k_dq, v_dq [E, S, Hkv, ctx, d] dequantised caches of the (expert, stream) pairs with
    lengths [E, S]; topk_idx, topk_w [S, k].  Default: out[s] = sum_j w[s,j] * attention(q[s], pair(e_j, s)),
    the expert-parallel combine of core/distributed/distributed_pikv.py:174-194 (expert output times routing
    weight, summed over the experts, i.e. over the ranks) with decode_attention as the expert's read of its
    cache.  lse_merge=True instead merges the k attentions as one softmax over the union of the k caches
    (no counterpart in the reference).  Returns out [S, Hq, d] fp32."""
    q = np.asarray(q, F32)
    S, Hq, d = q.shape
    k = topk_idx.shape[1]
    out = np.zeros((S, Hq, d), F32)
    for s in range(S):
        os_, ls_ = [], []
        for j in range(k):
            e = int(topk_idx[s, j])
            n = int(lengths[e, s])
            if n == 0:
                os_.append(np.zeros((Hq, d), F32))
                ls_.append(np.full(Hq, -np.inf, F32))
                continue
            o, _ = decode_attention(q[s:s + 1], k_dq[e, s:s + 1], v_dq[e, s:s + 1], np.array([n]))
            g = Hq // k_dq.shape[2]
            lse = np.zeros(Hq, F32)
            for h in range(Hq):
                sc = (q[s, h] @ np.asarray(k_dq[e, s, h // g, :n], F32).T) / F32(math.sqrt(d))
                lse[h] = np.log(np.exp(sc - sc.max()).sum()) + sc.max()
            os_.append(o[0])
            ls_.append(lse)
        if lse_merge:
            L = np.stack(ls_)                                   # [k, Hq]
            m = L.max(axis=0)
            wgt = np.where(np.isfinite(L), np.exp(L - np.where(np.isfinite(m), m, 0)[None]), 0)
            den = wgt.sum(axis=0)
            for j in range(k):
                out[s] += os_[j] * (wgt[j] / np.where(den > 0, den, 1))[:, None]
        else:
            for j in range(k):
                out[s] += os_[j] * F32(topk_w[s, j])
    return out


def rope_tables(max_pos: int, dim: int):
    """cos / sin [max_pos, dim/2] of RotaryEmbedding._compute_cos_sin_cache, core/single/pikv_attention.py:349-367
    (numpy's cos / sin may differ from torch's in the last bit: parity tests pass the reference's own tables)."""
    position = np.arange(max_pos, dtype=F32)[:, None]
    freq = (F32(1.0) / (F32(10000.0) ** (np.arange(0, dim, 2, dtype=F32) / F32(dim)))).astype(F32)
    pf = (position * freq).astype(F32)
    return np.cos(pf).astype(F32), np.sin(pf).astype(F32)


def rope_rotate(x, positions, cos, sin):
    """RotaryEmbedding.forward on one tensor, core/single/pikv_attention.py:369-400: x [T, heads, d]; the halves
    [..., :d/2] and [..., d/2:] rotate with cos / sin [positions]; every product and sum rounded to fp32."""
    x = np.asarray(x, F32)
    d = x.shape[-1]
    c = np.asarray(cos, F32)[np.asarray(positions)][:, None, :]
    s = np.asarray(sin, F32)[np.asarray(positions)][:, None, :]
    top, bot = x[..., : d // 2], x[..., d // 2:]
    out_top = ((top * c).astype(F32) + ((-bot) * s).astype(F32)).astype(F32)
    out_bot = ((bot * c).astype(F32) + (top * s).astype(F32)).astype(F32)
    return np.concatenate([out_top, out_bot], axis=-1)
