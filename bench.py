"""Benchmark of the routed KV-cache hot path: KV tokens/s for route + int8 quantise + append.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass over one batch of synthetic tokens: fused gate (logits of the
gate net's last layer, softmax, top-2, counts, slots) then the routed, quantised
append into the paged per-expert cache.  Workload at one GPU: 16384 tokens, hidden
4096, 8 experts top-2, 8 KV heads x 128, int8 symmetric per (token, head) group,
16-token pages; K/V ~ N(0,1) with 1% of channels scaled x20.  Data is synthetic.

Prints ONE JSON line (rank 0).  `value` is device-resident throughput, `e2e` the
same step through the public API with pinned host inputs copied in and the routing
result read back inside the timed region.  `--impl reference` times the CPU port of
the reference's arithmetic (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "kv_tokens_per_s_route_quant_append"
UNIT = "tokens/s"
WORKLOAD = dict(workload="route+int8-quant+append", tokens=16384, hidden=4096, experts=8, top_k=2, kv_heads=8,
                head_dim=128, page_tokens=16, quant="int8-sym-g128", capacity_factor=1.5)
GATE_BYTES_PER_TOKEN = 4096 * 2 + 8 * 4 + 3 * 2 * 4                      # act in; probs, idx, w, slot out
APPEND_BYTES_PER_TOKEN = 2 * 1024 * 2 + 16 + 2 * 2 * 1024 + 2 * 16 * 2   # K,V in; idx/slot; 2 copies of codes + scales
APPEND_BYTES_INT4 = 2 * 1024 * 2 + 16 + 2 * 2 * 512 + 2 * 16 * (2 + 4)   # 4-bit codes, bf16 scales, fp32 zero points
# DRAM bytes per launch (read + write) at 16384 tokens, from the ncu captures summarised under profiles/
# (the append's 67.4 MB of reads arrive in full; of its 68 MB of writes 21.6 MB had left the 126 MB L2 at kernel end)
TRAFFIC = {"gate": 139.2e6, "append": 89.0e6}


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        if os.environ.get("PIKV_BENCH_NO_CLOCKS") == "1":      # testing aid: run without the nvidia-smi poller
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()     # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def synth_inputs(T, H, E, kv_dim, seed, device=None, pin=False):
    import torch
    g = torch.Generator().manual_seed(seed)
    act = torch.randn(T, H, generator=g).bfloat16()
    K = torch.randn(T, kv_dim, generator=g)
    V = torch.randn(T, kv_dim, generator=g)
    cols = torch.randperm(kv_dim, generator=g)[: round(0.01 * kv_dim)]
    K[:, cols] *= 20.0
    V[:, cols] *= 20.0
    K, V = K.bfloat16(), V.bfloat16()
    if pin:
        return act.pin_memory(), K.pin_memory(), V.pin_memory()
    if device is not None:
        return act.to(device), K.to(device), V.to(device)
    return act, K, V


def gate_weights(H, E, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    bound = 1.0 / H ** 0.5                                   # nn.Linear default (Kaiming uniform, a=sqrt(5))
    w2 = (torch.rand(E, H, generator=g) * 2 - 1) * bound
    b2 = (torch.rand(E, generator=g) * 2 - 1) * bound
    return w2.bfloat16(), b2


# ----------------------------------------------------------------------------- CPU port (reference arm)
def host_threads():
    """Threads the CPU port may use: the cores this process is allowed on.  torchrun exports OMP_NUM_THREADS=1
    for its workers; the port is a baseline of the host, so it lifts that limit for itself (before numpy
    loads its BLAS)."""
    try:
        n = len(os.sched_getaffinity(0))
    except Exception:
        n = os.cpu_count() or 1
    return max(1, n)


class CpuPort:
    """The numpy port of one step, with its cache arrays allocated once (int8 codes, fp32 scales).  The gate
    GEMM is BLAS (threaded); the element-wise parts (softmax / top-k, the per-slice quantisation, the scatter of
    the rows into the cache) are numpy calls that release the GIL, run over token chunks on `nthreads` threads;
    the slot scan is serial."""

    def __init__(self, tokens, nthreads):
        from concurrent.futures import ThreadPoolExecutor
        import numpy as np
        cfg = WORKLOAD
        self.H, self.E, self.k = cfg["hidden"], cfg["experts"], cfg["top_k"]
        kv = cfg["kv_heads"] * cfg["head_dim"]
        act, K, V = synth_inputs(tokens, self.H, self.E, kv, 1)
        w2, b2 = gate_weights(self.H, self.E, 7)
        self.a, self.K, self.V = act.float().numpy(), K.float().numpy(), V.float().numpy()
        self.w, self.b = w2.float().numpy(), b2.numpy()
        self.cap = int(tokens * cfg["capacity_factor"] * self.k / self.E)
        self.T, self.n = tokens, nthreads
        self.pool = ThreadPoolExecutor(nthreads)
        self.bounds = [(i * tokens // nthreads, (i + 1) * tokens // nthreads) for i in range(nthreads)]
        G = kv // 128
        self.codes = [np.zeros((self.E, self.cap, kv), np.int8) for _ in range(2)]
        self.scales = [np.zeros((self.E, self.cap, G), np.float32) for _ in range(2)]

    def step(self):
        from oracle import pikv_oracle as O
        import numpy as np
        logits = O.gate_logits(self.a, self.w, self.b)
        tails = list(self.pool.map(lambda ab: O.gate_tail(logits[ab[0]:ab[1]], self.k), self.bounds))
        idx = np.concatenate([t[1] for t in tails])
        slot, counts_k = O.slot_assign_fast(idx, self.E, self.cap)

        def chunk(ab):
            lo, hi = ab
            t_ix, j_ix = np.nonzero(slot[lo:hi] >= 0)
            e, sl = idx[lo:hi][t_ix, j_ix], slot[lo:hi][t_ix, j_ix]
            for x, codes, scales in ((self.K, self.codes[0], self.scales[0]), (self.V, self.codes[1], self.scales[1])):
                q, sc, _ = O.quant_token_groups(x[lo:hi], 8, 128, True)
                codes[e, sl] = q[t_ix].astype(np.int8)
                scales[e, sl] = sc[t_ix]

        list(self.pool.map(chunk, self.bounds))
        return counts_k

    def close(self):
        self.pool.shutdown()


def run_cpu(steps, warmup, tokens):
    nthreads = host_threads()
    for var in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "OPENBLAS_NUM_THREADS"):
        os.environ[var] = str(nthreads)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(nthreads)
    except Exception:
        pass
    port = CpuPort(tokens, nthreads)
    for _ in range(warmup):
        port.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        port.step()
    dt = (time.perf_counter() - t0) / steps
    port.close()
    return tokens / dt, dt, nthreads


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # every step is one full 16384-token batch (about 0.1-0.4 s on the host); the step count is the caller's,
    # cut only where the run would pass a few minutes
    steps, warmup = max(1, min(args.steps, 200)), max(1, min(args.warmup, 3))
    tokens = WORKLOAD["tokens"]
    value, dt, cores = run_cpu(steps, warmup, tokens)
    sample = (f"{steps} full batches of {tokens} tokens (numpy port of the reference arithmetic; BLAS GEMM and "
              f"token-chunked element-wise parts on {cores} threads)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": dict(WORKLOAD),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def pool_hash(t):
    """Order-sensitive 64-bit checksum of a pool tensor (wrapping int64 arithmetic, computed on its device)."""
    import torch
    raw = t.contiguous().view(torch.uint8).view(-1)
    pad = (-raw.numel()) % 8
    if pad:
        raw = torch.cat([raw, raw.new_zeros(pad)])
    w = raw.view(torch.int64)
    pos = torch.arange(w.numel(), device=w.device, dtype=torch.int64)
    return int(((w ^ (pos * 0x1E3779B97F4A7C15)) * (2 * pos + 1)).sum().item())


def parity_single(torch, pikv_b200, ops, dev, cfg, w2, b2):
    """One fixed-seed config-2 step at full size against the oracle, outside every timed region: expert
    indices (mismatches must be near-ties of the oracle's top-k and are counted), then - on the GPU's own
    indices - slots, per-column counts, lengths, every code and every stored scale, bit for bit."""
    import numpy as np
    from oracle import pikv_oracle as O
    T, H, E, k = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["top_k"]
    n_kv = cfg["kv_heads"]
    kv = n_kv * cfg["head_dim"]
    cap = int(T * cfg["capacity_factor"] * k / E)
    act, K, V = synth_inputs(T, H, E, kv, 0)
    g = ops.gate_fused(act.to(dev), w2, b2, top_k=k, capacity=cap)
    cache = pikv_b200.PagedKVCache(E, cap, n_kv, device=dev)
    cache.append(K.to(dev), V.to(dev), g.topk_idx, g.slot)
    torch.cuda.synchronize()
    cache.check_status()
    logits = O.gate_logits(act.float().numpy(), w2.float().cpu().numpy(), b2.cpu().numpy())
    probs, idx, tw = O.gate_tail(logits, k)
    gi = g.topk_idx.cpu().numpy()
    diff = (gi != idx).any(axis=1)
    margin = O.topk_margin(probs, k)
    rec = {"n": 1, "tokens": T, "idx_mismatch": int(diff.sum()), "idx_near_ties": int((diff & (margin < 1e-4)).sum())}
    ok = rec["idx_mismatch"] == rec["idx_near_ties"]
    rec["probs_max_abs_err"] = float(np.abs(g.probs.cpu().numpy() - probs).max())
    ok &= rec["probs_max_abs_err"] < 1e-3          # bf16 products, fp32 accumulation in another order
    slot, counts_k = O.slot_assign_fast(gi, E, cap)
    same = lambda a_, b_: "bit-exact" if np.array_equal(a_, b_) else "MISMATCH"
    rec["slots"] = same(g.slot.cpu().numpy(), slot)
    rec["counts"] = same(g.counts_k.cpu().numpy(), counts_k)
    ref = O.routed_append(K.float().numpy(), V.float().numpy(), gi, slot, E, cap, 8, True, 128)
    rec["lengths"] = same(g.new_len.cpu().numpy(), ref["length"])
    lens = ref["length"]
    seq = np.repeat(np.arange(E), cap).astype(np.int32)
    pos = np.tile(np.arange(cap), E).astype(np.int32)
    valid = pos < lens[seq]
    seq_t, pos_t = torch.from_numpy(seq[valid]).to(dev), torch.from_numpy(pos[valid]).to(dev)
    mp = cache.max_pages
    for name in ("k", "v"):
        _, codes = cache.gather(seq_t, pos_t, name, codes=True)
        rec[f"{name}_codes"] = same(codes.cpu().numpy(), ref[f"{name}_codes"][seq[valid], pos[valid]].astype(np.int8))
        sc = getattr(cache, f"{name}_scale").view(E, mp, n_kv, 16).permute(0, 1, 3, 2).reshape(E, mp * 16, n_kv)[:, :cap]
        got = sc.float().cpu().numpy()[seq[valid], pos[valid]]
        rec[f"{name}_scales"] = same(got, O.bf16_round(ref[f"{name}_scale"][seq[valid], pos[valid]]))
    rec["rows_checked"] = int(valid.sum())
    ok &= all(v != "MISMATCH" for v in rec.values())
    rec["ok"] = bool(ok)
    return rec


def parity_multi(torch, dist, pikv_b200, ops, dev, rank, world, cfg, w2, b2, mode):
    """The ranks' caches after one fixed-seed step against the cache ONE GPU builds from the concatenated
    batch: every rank checksums its pools, rank 0 routes all world x tokens on its own GPU and compares its
    slices (expert block r) and lengths with rank r's."""
    from pikv_b200 import distributed as pd
    T, H, E, k = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["top_k"]
    n_kv = cfg["kv_heads"]
    kv = n_kv * cfg["head_dim"]
    cap = int(T * world * cfg["capacity_factor"] * k / E)
    act, K, V = synth_inputs(T, H, E, kv, 5000 + rank, device=dev)
    shard = (pd.PeerShardedKVCache if mode == "peer" else pd.ExpertShardedKVCache)(E, cap, n_kv, dev)
    shard.route_append(act, w2, b2, K, V, top_k=k)
    torch.cuda.synchronize()
    dist.barrier()
    status = int(shard.cache.status.item())
    names = ("k_codes", "v_codes", "k_scale", "v_scale", "length")
    mine = torch.tensor([pool_hash(getattr(shard.cache, n)) for n in names] + [status], dtype=torch.int64, device=dev)
    allh = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    rec = None
    if rank == 0:
        parts = [synth_inputs(T, H, E, kv, 5000 + r, device=dev) for r in range(world)]
        A, KK, VV = (torch.cat([p_[i] for p_ in parts]) for i in range(3))
        g = ops.gate_fused(A, w2, b2, top_k=k, capacity=cap)
        single = pikv_b200.PagedKVCache(E, cap, n_kv, device=dev)
        single.append(KK, VV, g.topk_idx, g.slot)
        single.length.copy_(g.new_len)
        torch.cuda.synchronize()
        single.check_status()
        per, pages = E // world, single.max_pages
        bad = []
        for r in range(world):
            sl = slice(r * per * pages, (r + 1) * per * pages)
            want = [pool_hash(getattr(single, n)[sl]) for n in names[:4]] + [pool_hash(single.length[r * per:(r + 1) * per]), 0]
            got = [int(x) for x in allh[r].tolist()]
            bad += [f"rank{r}:{n}" for n, w_, g_ in zip(names + ("status",), want, got) if w_ != g_]
        rec = {"n": world, "tokens": T * world, "against": "the cache one GPU builds from the concatenated batch",
               "codes": "bit-exact" if not any("codes" in b_ for b_ in bad) else "MISMATCH",
               "scales": "bit-exact" if not any("scale" in b_ for b_ in bad) else "MISMATCH",
               "lengths": "equal" if not any("length" in b_ for b_ in bad) else "MISMATCH",
               "status_words": "clear" if not any("status" in b_ for b_ in bad) else "SET", "bad": bad, "ok": not bad}
        del single, parts, A, KK, VV
    del shard
    torch.cuda.empty_cache()
    return rec


def gpu_arm(args):
    import torch
    import torch.distributed as dist
    import pikv_b200
    from pikv_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU port")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    pikv_b200.lib()

    cfg = dict(WORKLOAD)
    app_bytes = APPEND_BYTES_PER_TOKEN
    if args.bits == 4:
        # config 2's second format: 4-bit asymmetric codes, bf16 scales and fp32 zero points per (token, head)
        cfg.update(workload="route+int4-quant+append", quant="int4-asym-g128")
        app_bytes = APPEND_BYTES_INT4
    T, H, E, k = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["top_k"]
    n_kv = cfg["kv_heads"]
    kv = n_kv * cfg["head_dim"]
    w2, b2 = gate_weights(H, E, 7)
    w2, b2 = w2.to(dev), b2.to(dev)
    steps, warmup = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(fn):
        """CUDA graph of the C-ABI calls `fn` makes (they allocate nothing and never synchronise)."""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = pikv_b200.launch_count()
        with torch.cuda.graph(graph):
            fn()
        return graph, pikv_b200.launch_count() - n0

    def capture_pipelined(w, n):
        """One graph of n consecutive steps of the software-pipelined schedule, starting at buffer set 0:
        the gates' scoring kernels run back to back on a side stream, their slot finalisations on a second
        one, the appends on the capture stream; append(i) waits for gate(i), gate(i) for the append that
        last used its buffer set.  gate(0) ran before the graph (the previous
        replay issued it), gate(n) is issued for the next replay, so a replay holds n gates and n appends
        and one kernel's ramp-up and tail fill with the other's traffic.  n must be a multiple of the
        number of buffer sets, or the last window of the run."""
        R = w["R"]
        side, fin = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        for i in range(R):
            w["score"](i)                # allocates each result's own gate workspace before the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = pikv_b200.launch_count()
        with torch.cuda.graph(graph):
            cur = torch.cuda.current_stream()
            side.wait_stream(cur)
            appended = []
            for i in range(n):
                if i + 1 - R >= 0:
                    side.wait_event(appended[i + 1 - R])       # buffer set (i+1) % R is free again
                with torch.cuda.stream(side):
                    w["score"]((i + 1) % R)                    # pikv_gate_fused, phase 1: the scoring kernel
                    scored = torch.cuda.Event()
                    scored.record(side)
                fin.wait_event(scored)
                with torch.cuda.stream(fin):
                    w["slots"]((i + 1) % R)                    # phase 2: the short slot finalisation
                    gated = torch.cuda.Event()
                    gated.record(fin)
                w["pappend"](i % R)                            # pikv_kv_append_quant
                ev = torch.cuda.Event()
                ev.record(cur)
                appended.append(ev)
                cur.wait_event(gated)                          # append(i+1) needs gate(i+1)
            cur.wait_stream(side)
            cur.wait_stream(fin)
        return graph, pikv_b200.launch_count() - n0

    def run_pipelined(w, window, tail):
        """replay(i) for timed(): step i is the first of a window -> replay that window's graph."""
        def replay(i, total):
            if i % window[2] == 0:
                (window if total - i >= window[2] else tail)[0].replay()
        return replay

    def timed(replay, n, hooks=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        if hooks:
            hooks["begin"]()      # side streams start after the start event
        for i in range(n):
            replay(i)
        if hooks:
            hooks["end"]()        # and the stop event waits for them
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    def timed_repeats(replay, n, hooks=None, min_total_ms=500.0, min_reps=10, max_reps=600):
        """The K-step timed region, repeated: the headline is the median region, the spread is reported.  The
        repeat count comes from the first region (max over ranks, so every rank runs the same number) and is
        at least `min_reps`; repeating until `min_total_ms` also gives the clock sampler (one sample per
        100 ms) something to see."""
        first = timed(replay, n, hooks)
        if world > 1:
            f = torch.tensor([first], device=dev)
            dist.all_reduce(f, op=dist.ReduceOp.MAX)
            first = float(f.item())
        reps = int(min(max_reps, max(min_reps, min_total_ms / max(first, 1e-3))))
        out = [timed(replay, n, hooks) for _ in range(reps)]
        if world > 1:
            t_ = torch.tensor(out, device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)      # every region: the slowest rank's time
            out = [float(x) for x in t_.tolist()]
        return out

    def single_gpu_workload(tokens, bits=None):
        """R rotating input sets and caches so that no step finds its inputs in L2 (one set is 201 MB at
        16384 tokens, L2 is 126 MB)."""
        bits = args.bits if bits is None else bits
        cap = int(tokens * cfg["capacity_factor"] * k / E)
        R = 6 if tokens <= 32768 else 3     # more sets in flight let the gates run further ahead of the appends
        sets = [synth_inputs(tokens, H, E, kv, 100 + i, device=dev) for i in range(R)]
        caches = [pikv_b200.PagedKVCache(E, cap, n_kv, bits=bits, symmetric=(bits == 8), device=dev) for _ in range(R)]
        outs = [ops.gate_fused(sets[0][0], w2, b2, top_k=k, capacity=cap, want_probs=True) for _ in range(R)]

        def gate(i):
            return ops.gate_fused(sets[i][0], w2, b2, top_k=k, capacity=cap, out=outs[i])

        def append(i):
            caches[i].append(sets[i][1], sets[i][2], outs[i].topk_idx, outs[i].slot)

        def step(i):
            # one call: the gate kernel, then the append kernel that also finishes the slot scan
            caches[i].route_append(sets[i][0], w2, b2, sets[i][1], sets[i][2], top_k=k, capacity=cap, out=outs[i])

        def score(i):
            return ops.gate_fused(sets[i][0], w2, b2, top_k=k, capacity=cap, out=pouts[i], phase=1)

        def slots(i):
            return ops.gate_fused(sets[i][0], w2, b2, top_k=k, capacity=cap, out=pouts[i], phase=2)

        def pappend(i):
            caches[i].append(sets[i][1], sets[i][2], pouts[i].topk_idx, pouts[i].slot)

        # results of the pipelined schedule: each owns its gate workspace (several batches are in flight)
        pouts = [ops.gate_fused(sets[0][0], w2, b2, top_k=k, capacity=cap, want_probs=True) for _ in range(R)]
        return dict(R=R, cap=cap, sets=sets, caches=caches, outs=outs, gate=gate, append=append, step=step,
                    score=score, slots=slots, pappend=pappend)

    def kernel_times(w, n):
        """Average device time per launch of the gate's scoring kernel, of its slot finalisation and of the
        append: each kernel is captured R times back to back (one launch per buffer set, so every launch
        reads cold inputs) and the graph is timed with events on the launching stream."""
        R_ = w["R"]
        out = []
        for name in ("score", "slots", "pappend"):
            for i in range(R_):
                w["score"](i)                              # valid gate state for the later phases
                if name == "pappend":
                    w["slots"](i)                          # the append is timed on final slots
            graph = capture(lambda: [w[name](i) for i in range(R_)])[0]
            reps = max(20, -(-n // R_))
            graph.replay()
            out.append(timed(lambda i: graph.replay(), reps) / (reps * R_))
        return out

    roof = e2e = cpu = large = parity = extras = None
    multi = {}
    if world > 1:
        from pikv_b200 import distributed as pd
        parity = parity_multi(torch, dist, pikv_b200, ops, dev, rank, world, cfg, w2, b2, args.shard_mode)
        step_fn, extra_cfg = pd.make_bench_step(dev, rank, world, cfg, w2, b2, synth_inputs, mode=args.shard_mode)
        R = extra_cfg.pop("buffer_sets", 1)
        hooks = extra_cfg.pop("hooks", None)
        verify = extra_cfg.pop("verify", None)
        # Untimed blocks of steps for `warm_s` seconds before the timed regions; every rank stops after the same
        # block (the decision comes from the all-reduced clock).  The JSON line states the seconds.  (Measured with
        # 0, 8 and 45 s: the same step time, so a few seconds are the default.)
        warm_s = float(os.environ.get("PIKV_BENCH_MULTI_WARMUP_S", str(args.multi_warmup_s)))
        t_begin, base, block = time.time(), steps, 2000
        while warm_s > 0:
            hooks["begin"]() if hooks else None
            for i in range(block):
                step_fn(base + i)                 # indices past the timed range
            hooks["end"]() if hooks else None
            torch.cuda.synchronize()
            tb = torch.tensor([time.time() - t_begin], device=dev)
            dist.all_reduce(tb, op=dist.ReduceOp.MAX)
            base += block
            if float(tb[0]) > warm_s:
                break
        multi["warmup_s"] = round(time.time() - t_begin, 1)
        launch_mode = "C-ABI calls only (gate, count exchange + plan, sharded append, scale push), one CUDA graph per lane step" \
            if args.shard_mode == "peer" else "eager C-ABI calls + NCCL all_to_all"
        per_step = extra_cfg.pop("launches_per_step", None)     # kernels inside a replayed graph
        replay = step_fn
        for i in range(warmup):
            replay(i)
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        n0 = pikv_b200.launch_count()
        regions = timed_repeats(replay, steps, hooks, min_total_ms=500.0)
        ms = median(regions)
        launches = per_step * steps if per_step is not None else (pikv_b200.launch_count() - n0) // (len(regions) + 1)
        clocks = sampler.stop() if rank == 0 else None
        if verify is not None:
            multi["lanes_verified"] = verify()               # status words and lengths of every lane's cache
        link = extra_cfg.pop("link_bytes_per_step", None)
        if link is not None:
            multi["link_bytes_per_gpu_per_step"] = link
            multi["link_GBps_per_gpu"] = link / (ms / steps * 1e-3) / 1e9
        e2e_io = extra_cfg.pop("e2e_io", None)
        if e2e_io is not None:
            e2e_step, h2d, d2h = e2e_io
            for i in range(R):
                e2e_step(i)
            e2e_ms = torch.tensor([timed(e2e_step, steps, hooks)], device=dev)
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
            e2e = {"value": T * world * steps / (float(e2e_ms.item()) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                   "d2h_bytes_per_step": d2h * world, "ms_per_step": float(e2e_ms.item()) / steps}
    else:
        parity = parity_single(torch, pikv_b200, ops, dev, cfg, w2, b2) if args.bits == 8 else None
        wl = single_gpu_workload(T)
        R = wl["R"]
        # serial schedule: one stream, gate then append (pikv_route_append), one graph per step
        graphs = [capture(lambda i=i: wl["step"](i)) for i in range(R)]
        for i in range(warmup):
            graphs[i % R][0].replay()
        serial_ms = median(timed_repeats(lambda i: graphs[i % R][0].replay(), steps, min_total_ms=100.0)) / steps
        sampler = ClockSampler(local)
        if args.schedule == "pipelined":
            # batch i+1 is gated while batch i is appended; K replays = K gates + K appends
            W = 2 * R
            window = capture_pipelined(wl, W) + (W,)
            tail = capture_pipelined(wl, steps % W) + (steps % W,) if steps % W else window
            wl["score"](0), wl["slots"](0)
            for i in range(max(1, warmup // W)):
                window[0].replay()
            sampler.start()
            replay = run_pipelined(wl, window, tail)
            regions = timed_repeats(lambda i: replay(i, steps), steps)
            launches = window[1] * (steps // W) + (tail[1] if steps % W else 0)
            launch_mode = (f"CUDA graphs of {W} steps (captured C-ABI calls): gates on one stream, appends on another, "
                           "append(i) after gate(i)")
        else:
            sampler.start()
            regions = timed_repeats(lambda i: graphs[i % R][0].replay(), steps)
            launches = graphs[0][1] * steps
            launch_mode = "one CUDA graph replay per step (captured C-ABI calls, one stream)"
        ms = median(regions)
        clocks = sampler.stop()
        extra_cfg = {"parallelism": "single", "schedule": args.schedule}
    ms_max = ms
    value = T * world * steps / (ms_max * 1e-3)
    repeats = {"regions": len(regions), "steps_per_region": steps, "timed_ms_total": sum(regions),
               "ms_per_step_median": ms / steps, "ms_per_step_min": min(regions) / steps, "ms_per_step_max": max(regions) / steps}

    if world == 1:
        peak, peak_src = measured_peak_gbs()
        gate_ms, fin_ms, app_ms = kernel_times(wl, steps)
        gate_gbs = GATE_BYTES_PER_TOKEN * T / (gate_ms * 1e-3) / 1e9
        app_gbs = app_bytes * T / (app_ms * 1e-3) / 1e9
        step_gbs = (GATE_BYTES_PER_TOKEN + app_bytes) * T / (ms_max / steps * 1e-3) / 1e9
        dom = "gate" if gate_ms >= app_ms else "append"
        roof = {"bound": "hbm",
                "kernel": "gate_tc_kernel" if dom == "gate" else "kv_append_quant_kernel",
                "achieved": gate_gbs if dom == "gate" else app_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                "frac": (gate_gbs if dom == "gate" else app_gbs) / peak, "traffic": TRAFFIC.get(dom),
                "gate": {"ms": gate_ms, "GBps": gate_gbs, "frac": gate_gbs / peak, "bytes_per_token": GATE_BYTES_PER_TOKEN},
                "append": {"ms": app_ms, "GBps": app_gbs, "frac": app_gbs / peak, "bytes_per_token": app_bytes},
                "finalize": {"ms": fin_ms},
                "step": {"GBps": step_gbs, "frac": step_gbs / peak},
                "serial_step": {"GBps": (GATE_BYTES_PER_TOKEN + app_bytes) * T / (serial_ms * 1e-3) / 1e9,
                                "frac": (GATE_BYTES_PER_TOKEN + app_bytes) * T / (serial_ms * 1e-3) / 1e9 / peak}}

        # end to end: pinned host inputs copied in, routing result read back, every step (eager calls)
        cap, caches, outs = wl["cap"], wl["caches"], wl["outs"]
        h_sets = [synth_inputs(T, H, E, kv, 200 + i, pin=True) for i in range(2)]
        d_in = [tuple(torch.empty_like(x, device=dev) for x in h_sets[0]) for _ in range(2)]
        h_out = [torch.empty(T, k, dtype=torch.int32).pin_memory(), torch.empty(T, k, dtype=torch.float32).pin_memory(),
                 torch.empty(T, k, dtype=torch.int32).pin_memory(), torch.empty(E, dtype=torch.int32).pin_memory()]

        def e2e_step(i):
            src, dst = h_sets[i % 2], d_in[i % 2]
            for s_, d_ in zip(src, dst):
                d_.copy_(s_, non_blocking=True)
            g = ops.gate_fused(dst[0], w2, b2, top_k=k, capacity=cap, out=outs[i % R])
            caches[i % R].append(dst[1], dst[2], g.topk_idx, g.slot)
            h_out[0].copy_(g.topk_idx, non_blocking=True)
            h_out[1].copy_(g.topk_w, non_blocking=True)
            h_out[2].copy_(g.slot, non_blocking=True)
            h_out[3].copy_(g.new_len, non_blocking=True)

        for i in range(3):
            e2e_step(i)
        e2e_ms = timed(e2e_step, steps)
        h2d = sum(x.numel() * x.element_size() for x in h_sets[0])
        d2h = sum(x.numel() * x.element_size() for x in h_out)
        e2e = {"value": T * steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms / steps}
        for c in caches:
            c.check_status()
        assert pikv_b200.lib().pikv_gate_error_state() == 0, "a bounded wait in the gate kernel ran out"
        del wl, graphs, h_sets, d_in, caches, outs
        window = tail = None
        torch.cuda.empty_cache()

        if not args.no_large:
            # the same step at 8x the tokens: launch overhead and tail effects no longer matter
            T8 = 8 * T
            w8 = single_gpu_workload(T8)
            steps8 = max(3, steps // 4)
            if args.schedule == "pipelined":
                W8 = w8["R"]
                steps8 = -(-steps8 // W8) * W8
                win8 = capture_pipelined(w8, W8) + (W8,)
                w8["score"](0), w8["slots"](0)
                win8[0].replay()
                replay8 = run_pipelined(w8, win8, win8)
                ms8 = timed(lambda i: replay8(i, steps8), steps8)
                g8 = win8
            else:
                g8 = [capture(lambda i=i: w8["step"](i))[0] for i in range(w8["R"])]
                for i in range(3):
                    g8[i % w8["R"]].replay()
                ms8 = timed(lambda i: g8[i % w8["R"]].replay(), steps8)
            gate8, _, app8 = kernel_times(w8, steps8)
            large = {"tokens": T8, "value": T8 * steps8 / (ms8 * 1e-3), "unit": UNIT, "ms_per_step": ms8 / steps8,
                     "gate_frac": GATE_BYTES_PER_TOKEN * T8 / (gate8 * 1e-3) / 1e9 / peak,
                     "append_frac": app_bytes * T8 / (app8 * 1e-3) / 1e9 / peak,
                     "step_frac": (GATE_BYTES_PER_TOKEN + app_bytes) * T8 / (ms8 / steps8 * 1e-3) / 1e9 / peak}
            del w8, g8
            torch.cuda.empty_cache()

        if not args.no_extras and args.bits == 8:
            extras = other_kernels(torch, pikv_b200, ops, dev, peak, peak_src, local, single_gpu_workload, kernel_times)

    sharded = None
    if not args.no_sharded and args.bits == 8:
        peak_s, _ = measured_peak_gbs()
        torch.cuda.empty_cache()
        sharded = sharded_arm(torch, dist, dev, rank, world, steps, local, peak_s)

    if world == 1 and not args.no_cpu_baseline:
        v, dt, cores = run_cpu(10, 2, T)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"10 full batches of {T} tokens on the host (numpy port of the reference arithmetic, {cores} threads)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_max / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": f"bf16 in, fp32 math, int{args.bits} codes", "data": "synthetic",
            "config": {**cfg, **extra_cfg, "l2": f"inputs larger than L2, rotated over {R} buffer sets"},
            "clocks": clocks, "repeats": repeats, "e2e": e2e, "gpu_launches": int(launches), "launch": launch_mode,
            "roofline": roof, "cpu_baseline": cpu, "parity": parity, "large_batch": large,
        }
        line.update(multi)
        if sharded is not None:
            line["sharded"] = sharded
        if world == 1:
            line["serial_schedule"] = {"ms_per_step": serial_ms, "value": T / (serial_ms * 1e-3), "unit": UNIT,
                                       "launch": "pikv_route_append on one stream, one graph per step"}
            if extras is not None:
                line["other_kernels"] = extras
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity.get("ok", False):
        raise SystemExit("parity check failed: " + json.dumps(parity))
    if sharded is not None and sharded.get("parity") is not None and not sharded["parity"]["ok"]:
        raise SystemExit("sharded parity check failed: " + json.dumps(sharded["parity"]))


def other_kernels(torch, pikv_b200, ops, dev, peak, peak_src, gpu_index, single_gpu_workload, kernel_times):
    """The rest of the metric at the sizes BASELINE.json names, as sub-records of the one JSON line: each is
    timed for about 0.6 s (CUDA events) with its own clock sample; `bytes` are algorithmic bytes per launch.
      decode           config 3: 64 streams x 32 query / 8 KV heads x context 32768, int8 cache
      decode_h2o       the same step with the H2O accumulated-attention update (scores out + accumulate)
      decode_int4      the same over the 4-bit asymmetric cache
      h2o_select / h2o_compact / decode_budgeted   eviction to the 2048-token budget and decode over it
      lowrank          config 4: 262144 x 1024 -> rank 64 / 32 / 16
      append_int4      config 2's second format (4-bit asymmetric) through the append kernel"""
    out = {}

    def measure(fn, launches_per_call=1, target_s=0.6):
        """Device time per call of fn, replayed as a CUDA graph (the short kernels here would otherwise be timed
        at the rate the host can launch them), for about target_s seconds with the clock sampler running."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        n = int(max(5, min(5000, target_s * 1e3 / max(e0.elapsed_time(e1), 1e-3))))
        sampler = ClockSampler(gpu_index)
        sampler.start()
        e0.record()
        for _ in range(n):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n, n, sampler.stop()

    def record(name, ms, n, clocks, nbytes, kernel, **more):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "bytes": nbytes, "GBps": gbs, "frac": gbs / peak, "peak": peak, "peak_source": peak_src,
                     "kernel": kernel, "launches_timed": n, "clocks": clocks, **more}

    B, n_q, n_kv, ctx = 64, 32, 8, 32768
    q = torch.randn(B, n_q, 128, device=dev).bfloat16()
    for bits in (8, 4):
        cache = fill_stream_cache(pikv_b200, torch, dev, B, n_kv, ctx, bits=bits)
        per_tok = 2 * 128 + 2 * 2 if bits == 8 else 2 * 64 + 2 * 2 + 2 * 4
        by = B * n_kv * ctx * per_tok + 2 * B * n_q * 128 * 2
        ms, n, cl = measure(lambda: cache.decode_attention(q))
        record("decode" if bits == 8 else "decode_int4", ms, n, cl, by, f"decode_attn_kernel<{bits}>",
               streams=B, context=ctx, context_tokens_per_s=B * ctx / (ms * 1e-3))
        cache.check_status()
        if bits == 8:
            # decode + H2O accumulate: acc[b, kv head, pos] += sum over the group's query heads of the attention
            # probability (4.497 GB of algorithmic traffic: the cache, q, out, and acc read + written)
            acc = torch.zeros(B * n_kv, ctx, device=dev)
            h2o_ws = cache.h2o_workspace(B, n_q, ctx)

            def step_h2o():
                cache.decode_attention_h2o(q, acc, h2o_ws)

            ms, n, cl = measure(step_h2o)
            record("decode_h2o", ms, n, cl, by + 2 * B * n_kv * ctx * 4, "decode_attn_kernel<8> + h2o_accumulate_probs_kernel",
                   note="f16 probabilities relative to their softmax step go through HBM between the two kernels "
                        "(2 x 134 MB, not counted as algorithmic)")
            del h2o_ws
            scores = torch.empty(B, n_q, ctx, device=dev)

            def step_h2o_fp32():
                _, lse = cache.decode_attention(q, scores=scores)
                ops.h2o_accumulate_attn(scores, lse, cache.length, n_kv, acc)

            ms, n, cl = measure(step_h2o_fp32)
            record("decode_h2o_fp32_scores", ms, n, cl, by + 2 * B * n_kv * ctx * 4, "decode_attn_kernel<8> + h2o_accumulate_attn_kernel",
                   note="the same update through raw fp32 scores (2 x 268 MB between the kernels)")
            del scores
            acc = torch.rand(B * n_kv, ctx, device=dev)
            ts = torch.arange(ctx, dtype=torch.float32, device=dev).repeat(B * n_kv, 1)
            acc[:, ctx - 256:] = 0.0        # the recent window holds no heavy hitter: every segment keeps exactly 2048
            ms, n, cl = measure(lambda: ops.h2o_select(acc, ts, 1792, 256, as_bool=False))
            record("h2o_select", ms, n, cl, 2 * 4 * ctx * B * n_kv + B * n_kv * (ctx + 2048 * 4), "h2o_select_stream_kernel",
                   segments=B * n_kv, length=ctx, heavy=1792, recent=256)
            _, keep, cnt = ops.h2o_select(acc, ts, 1792, 256, as_bool=False)
            dst = pikv_b200.PagedKVCache(B, ctx, n_kv, device=dev)      # same page-table width as the source
            dacc, dts = torch.zeros(B * n_kv, keep.shape[1], device=dev), torch.zeros(B * n_kv, keep.shape[1], device=dev)
            ms, n, cl = measure(lambda: cache.compact_into(dst, keep, cnt, True, acc, ts, dacc, dts))
            record("h2o_compact", ms, n, cl, 2 * B * n_kv * 2048 * (2 * 128 + 2 * 2 + 4 + 4), "h2o_compact_kernel",
                   segments=B * n_kv, kept=2048)
            dst.length.fill_(2048)
            ms, n, cl = measure(lambda: dst.decode_attention(q, max_ctx=2048))
            record("decode_budgeted", ms, n, cl, B * n_kv * 2048 * per_tok + 2 * B * n_q * 128 * 2, "decode_attn_kernel<8>",
                   streams=B, context=2048)
            cache.check_status()
            dst.check_status()
            del dst, acc, ts, dacc, dts
        del cache
        torch.cuda.empty_cache()

    M, K = 262144, 1024
    x = torch.randn(M, K, device=dev).bfloat16()
    for r in (64, 32, 16):
        w = torch.nn.init.orthogonal_(torch.empty(K, K))[:r].contiguous().to(dev).bfloat16()
        ms, n, cl = measure(lambda: ops.lowrank_project(x, w, None, relu=True))
        record(f"lowrank_r{r}", ms, n, cl, M * K * 2 + M * r * 2, "lowrank_gemm_kernel", rows=M, hidden=K, rank=r,
               TFLOPs=2.0 * M * K * r / (ms * 1e-3) / 1e12)
    assert pikv_b200.lib().pikv_lowrank_error_state() == 0
    del x
    torch.cuda.empty_cache()

    # the gate net's first layer fused with ReLU, the second layer and the gate tail (tensor-bound): [T,4096] x
    # [4096,4096] + [T,4096] x [4096,8]; beside it the same net as a library GEMM + ReLU followed by the gate kernel
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf_peak = float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        tf_peak = 1400.0
    Tn, Hn, En = WORKLOAD["tokens"], WORKLOAD["hidden"], WORKLOAD["experts"]
    gx = torch.randn(Tn, Hn, device=dev).bfloat16()
    gw1 = (torch.randn(Hn, Hn, device=dev) / Hn ** 0.5).bfloat16()
    gb1 = torch.zeros(Hn, device=dev)
    gw2, gb2 = gate_weights(Hn, En, 7)
    gw2, gb2 = gw2.to(dev), gb2.to(dev)
    capn = int(Tn * WORKLOAD["capacity_factor"] * WORKLOAD["top_k"] / En)
    gout = ops.gate_mlp_fused(gx, gw1, gb1, gw2, gb2, top_k=2, capacity=capn)
    flops = 2.0 * Tn * Hn * Hn + 2.0 * Tn * Hn * En
    ms, n, cl = measure(lambda: ops.gate_mlp_fused(gx, gw1, gb1, gw2, gb2, top_k=2, capacity=capn, out=gout))
    assert pikv_b200.lib().pikv_gate_error_state() == 0
    out["gate_net"] = {"ms": ms, "flops": flops, "TFLOPs": flops / (ms * 1e-3) / 1e12, "frac": flops / (ms * 1e-3) / 1e12 / tf_peak,
                       "peak": tf_peak, "peak_source": "measured (sustained bf16)", "bound": "tensor", "kernel": "gate_mlp_kernel",
                       "launches_timed": n, "clocks": cl, "tokens": Tn, "hidden": Hn}
    gb1h = gb1.bfloat16()

    def library_net():
        h = torch.relu(torch.nn.functional.linear(gx, gw1, gb1h))
        ops.gate_fused(h, gw2, gb2, top_k=2, capacity=capn, out=gout)

    ms_l, n_l, cl_l = measure(library_net)
    out["gate_net"]["library_gemm_plus_gate_ms"] = ms_l
    del gx, gw1, gout
    torch.cuda.empty_cache()

    w4 = single_gpu_workload(WORKLOAD["tokens"], bits=4)
    sampler = ClockSampler(gpu_index)
    sampler.start()
    _, _, app4 = kernel_times(w4, 2000)
    cl = sampler.stop()
    record("append_int4", app4, 2000, cl, APPEND_BYTES_INT4 * WORKLOAD["tokens"], "kv_append_quant_kernel<bf16,4,asym>",
           tokens=WORKLOAD["tokens"])
    for c in w4["caches"]:
        c.check_status()
    return out


# ----------------------------------------------------------------------------- expert-sharded configuration
SHARDED = dict(workload="expert-sharded striped KV cache: prefill append + one decode step", experts=64, top_k=2, hidden=4096,
               streams=256, context=16384, q_heads=32, kv_heads=8, head_dim=128, stripe=1024, zipf_exponent=1.1,
               quant="int8-sym-g128")


def sharded_inputs(torch, dev, cfg, slot):
    """One of four rotating buffer sets of a 16384-token prefill chunk: gate-net activations, K, V (seeded by the
    slot, so every rank count builds the same cache for stream s from set s % 4)."""
    g = torch.Generator(device=dev).manual_seed(7000 + slot)
    T, H, kv = cfg["context"], cfg["hidden"], cfg["kv_heads"] * cfg["head_dim"]
    act = torch.randn(T, H, generator=g, device=dev).bfloat16()
    K = torch.randn(T, kv, generator=g, device=dev).bfloat16()
    V = torch.randn(T, kv, generator=g, device=dev).bfloat16()
    return act, K, V


def sharded_gate(torch, dev, cfg):
    """Gate weights whose logits are log Zipf(1.1)[e] + N(0,1): unit-norm random rows (act ~ N(0,1)) and the log
    popularity as the bias."""
    from pikv_b200.striping import zipf_expert_logits
    g = torch.Generator().manual_seed(11)
    w = torch.randn(cfg["experts"], cfg["hidden"], generator=g)
    w = (w / w.norm(dim=1, keepdim=True)).bfloat16().to(dev)
    b = torch.from_numpy(zipf_expert_logits(cfg["experts"], cfg["zipf_exponent"])).to(dev)
    return w, b


def sharded_capacity(cfg):
    """Rows per pair by expert: 1.3 x the expected share of a stream's tokens that select the expert (top-2 of
    log Zipf + N(0,1), estimated from 65536 seeded draws), rounded up to whole stripes.  Router statistics size
    the page pools; rows past a pair's capacity are dropped like the reference's rows past the cache size."""
    import numpy as np
    from pikv_b200.striping import zipf_expert_logits
    rng = np.random.default_rng(5)
    E = cfg["experts"]
    lg = zipf_expert_logits(E, cfg["zipf_exponent"])[None] + rng.standard_normal((65536, E)).astype(np.float32)
    top = np.argsort(-lg, axis=1)[:, :cfg["top_k"]]
    share = np.bincount(top.ravel(), minlength=E) / 65536.0
    st = cfg["stripe"]
    return ((np.ceil(1.3 * share * cfg["context"] / st) + 1) * st).astype(np.int64)


def sharded_arm(torch, dist, dev, rank, world, steps, gpu_index, peak):
    """Config 5: 64 experts top-2, 256 decode streams x context 16384, Zipf(1.1)-skewed routing, the caches of the
    (expert, stream) pairs striped over the GPUs.  Total work is fixed (strong scaling).  Timed: the prefill (every
    stream's 16384 tokens gated from hidden 4096 and appended through pikv_kv_append_striped) and one decode step
    (post -> attend -> combine) replayed as a CUDA graph.  Parity: sample streams' decode output against a
    one-GPU cache of the same streams built on rank 0."""
    import numpy as np
    import pikv_b200
    from pikv_b200 import ops
    from pikv_b200.striping import StripedLayout
    from pikv_b200.striped_cache import StripedShardedKVCache
    cfg = dict(SHARDED)
    E, S, k, n_q, n_kv = cfg["experts"], cfg["streams"], cfg["top_k"], cfg["q_heads"], cfg["kv_heads"]
    perm = np.random.default_rng(3).permutation(E)
    cap = sharded_capacity(cfg)
    lay = StripedLayout(E, S, world, cfg["stripe"], perm)
    cache = StripedShardedKVCache.create(lay, n_kv, n_q, k, cap, dev)
    w2, b2 = sharded_gate(torch, dev, cfg)
    sets = [sharded_inputs(torch, dev, cfg, i) for i in range(4)]
    spr = cache.streams_per_rank
    T = cfg["context"]

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- prefill: this rank's streams, one 16384-token chunk each ----
    streams_here = list(range(rank * spr, (rank + 1) * spr))
    # six independent chains of streams on six CUDA streams: the gate of one stream's chunk overlaps the
    # append of another's (each chain has its own gate result; a stream's step touches only its own lengths).
    # One GPU, whole prefill: 18.4 / 17.5 / 17.4 / 16.9 ms with 2 / 3 / 4 / 6 chains.
    NB = 6
    branches = [torch.cuda.Stream(device=dev) for _ in range(NB)]
    outs = [ops.gate_fused(sets[0][0], w2, b2, top_k=k, capacity=0) for _ in range(NB)]

    def fill():
        cur = torch.cuda.current_stream()
        for b_, st_ in enumerate(branches):
            st_.wait_stream(cur)
            with torch.cuda.stream(st_):
                for s_ in streams_here[b_::NB]:
                    a_, K_, V_ = sets[s_ % 4]
                    cache.route_append(s_, K_, V_, act=a_, w2=w2, b2=b2, out=outs[b_])
        for st_ in branches:
            cur.wait_stream(st_)
        cache.barrier()

    fill()                                   # eager once (workspaces, launch path), then as one CUDA graph: the step
    sync_all()                               # is three kernels per stream and the host would otherwise bound it
    cache.check_status()
    fill_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(fill_graph):
        fill()
    cache.pair_len.zero_()
    sync_all()
    sampler = ClockSampler(gpu_index)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fill_graph.replay()
    e1.record()
    sync_all()
    fill_ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(fill_ms, op=dist.ReduceOp.MAX)
    cache.check_status()

    # ---- decode step ----
    g = torch.Generator(device=dev).manual_seed(99)
    q_all = torch.randn(S, n_q, 128, generator=g, device=dev).bfloat16()
    dl = (b2[None] + torch.randn(S, E, generator=g, device=dev)).contiguous()
    route = ops.gate_fused(logits=dl, top_k=k, capacity=0)
    sl = slice(rank * spr, (rank + 1) * spr)
    q_loc, idx_loc, w_loc = q_all[sl].contiguous(), route.topk_idx[sl].contiguous(), route.topk_w[sl].contiguous()
    out = torch.empty(spr, n_q, 128, dtype=torch.bfloat16, device=dev)
    cache.decode_step(q_loc, idx_loc, w_loc, out=out)
    sync_all()
    cache.check_status()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        cache.decode_step(q_loc, idx_loc, w_loc, out=out)
    for _ in range(3):
        graph.replay()
    sync_all()
    n_dec = max(steps, 50)
    regions = []
    for _ in range(5):
        sync_all()
        e0.record()
        for _ in range(n_dec):
            graph.replay()
        e1.record()
        sync_all()
        regions.append(e0.elapsed_time(e1) / n_dec)
    dec = torch.tensor(regions, device=dev)
    if world > 1:
        dist.all_reduce(dec, op=dist.ReduceOp.MAX)
    dec_ms = median([float(x) for x in dec.tolist()])
    clocks = sampler.stop() if rank == 0 else None
    cache.check_status()

    # ---- load and link bytes of the step, from the routing ----
    lens = torch.zeros(S, E, dtype=torch.int32, device=dev)
    lens[sl] = cache.pair_len
    if world > 1:
        dist.all_reduce(lens)
    lens_h, idx_h = lens.cpu().numpy(), route.topk_idx.cpu().numpy()
    row_bytes = 2 * n_kv * 128 + 2 * n_kv * 2                        # K and V codes + bf16 scales of one token
    load = np.zeros(world)
    q_sends = np.zeros(world)
    part_recv = np.zeros(world)
    for s_ in range(S):
        dests = set()
        for e_ in idx_h[s_]:
            for r_ in range(world):
                n_ = int(lay.local_len(e_, s_, lens_h[s_, e_], r_))
                load[r_] += n_
                if n_ > 0:
                    dests.add(r_)
                    if r_ != int(lay.home(s_)):
                        part_recv[int(lay.home(s_))] += n_q * (128 + 1) * 4
        q_sends[int(lay.home(s_))] += len(dests - {int(lay.home(s_))}) * n_q * 128 * 2
    total_bytes = float(load.sum()) * row_bytes + 2 * S * n_q * 128 * 2
    tokens_total = S * T

    # ---- parity: sample streams against a one-GPU cache of the same streams ----
    sample = sorted({0, 1, S // 2, S - 1})
    outs_all = [torch.empty_like(out) for _ in range(world)] if world > 1 else [out]
    if world > 1:
        dist.all_gather(outs_all, out)
    parity = None
    if rank == 0:
        full = torch.cat(outs_all).float()
        lay1 = StripedLayout(E, len(sample), 1, cfg["stripe"], perm)
        from pikv_b200.striped_cache import emulate_ranks
        one = emulate_ranks(lay1, n_kv, n_q, k, cap, dev)[0]
        for i, s_ in enumerate(sample):
            a_, K_, V_ = sets[s_ % 4]
            one.route_append(i, K_, V_, act=a_, w2=w2, b2=b2)
        sel = torch.tensor(sample, device=dev)
        ref = one.decode_step(q_all[sel].contiguous(), route.topk_idx[sel].contiguous(), route.topk_w[sel].contiguous())
        torch.cuda.synchronize()
        one.check_status()
        same_len = bool(torch.equal(one.pair_len, lens[sel]))
        err = float((full[sel] - ref.float()).abs().max() / ref.float().abs().max())
        parity = {"n": world, "streams_checked": sample, "against": "a one-GPU cache of the same streams",
                  "pair_lengths": "equal" if same_len else "MISMATCH", "decode_max_rel_err": err, "tolerance": 1e-2,
                  "ok": bool(same_len and err <= 1e-2)}
        del one
    rec = {"config": cfg, "n_gpus": world, "scaling": "strong",
           "prefill": {"ms_total": float(fill_ms.item()), "tokens": tokens_total,
                       "tokens_per_s": tokens_total / (float(fill_ms.item()) * 1e-3),
                       "ms_per_16384_token_step": float(fill_ms.item()) / spr,
                       "link_bytes_per_gpu": float(tokens_total) / world * k * row_bytes * (world - 1) / world},
           "decode": {"ms_per_step": dec_ms, "regions_ms": regions, "steps_per_region": n_dec, "bytes": total_bytes,
                      "GBps_aggregate": total_bytes / (dec_ms * 1e-3) / 1e9,
                      "frac_of_n_x_peak": total_bytes / (dec_ms * 1e-3) / 1e9 / (peak * world),
                      "streams_per_s": S / (dec_ms * 1e-3),
                      "hottest_to_mean_gpu_load": float(load.max() / load.mean()),
                      "link_bytes_per_gpu_max": float((q_sends + part_recv).max()),
                      "launch": "post, plan, decode_attn, return, combine: five kernels per rank, one CUDA graph"},
           "clocks": clocks, "parity": parity}
    del cache
    torch.cuda.empty_cache()
    return rec


# ----------------------------------------------------------------------------- secondary workloads
def fill_stream_cache(pikv_b200, torch, dev, B, n_kv, ctx, seed=0, bits=8):
    """int8-symmetric (or 4-bit asymmetric) cache of B streams x ctx tokens, written through the append
    kernel stream by stream."""
    cache = pikv_b200.PagedKVCache(B, ctx, n_kv, bits=bits, symmetric=(bits == 8), device=dev)
    g = torch.Generator(device=dev).manual_seed(seed)
    pos = torch.arange(ctx, dtype=torch.int32, device=dev)[:, None].contiguous()
    for b in range(B):
        K = torch.randn(ctx, n_kv * 128, generator=g, device=dev).bfloat16()
        V = torch.randn(ctx, n_kv * 128, generator=g, device=dev).bfloat16()
        cache.append(K, V, torch.full((ctx, 1), b, dtype=torch.int32, device=dev), pos)
    cache.length.fill_(ctx)
    return cache


def secondary_arm(args):
    """Decode attention / H2O select / low-rank projection at the sizes of the reference's headline configurations: one JSON line each,
    same keys as the main line (metric names differ)."""
    import torch
    import pikv_b200
    from pikv_b200 import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peak, peak_src = measured_peak_gbs()
    steps, warmup = args.steps, max(args.warmup, 3)

    def timed(fn, n):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def emit(metric, unit, value, ms, cfg, roof, launches):
        print(json.dumps({"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": steps, "warmup": warmup,
                          "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                          "data": "synthetic", "config": cfg, "roofline": roof, "gpu_launches": launches}))

    if args.workload == "decode":
        B, n_q, n_kv, ctx = args.streams, 32, 8, args.context
        cache = fill_stream_cache(pikv_b200, torch, dev, B, n_kv, ctx, bits=args.bits)
        q = torch.randn(B, n_q, 128, device=dev).bfloat16()
        n0 = pikv_b200.launch_count()
        ms = timed(lambda: cache.decode_attention(q, splits=args.splits), steps)
        launches = (pikv_b200.launch_count() - n0) * steps // (steps + warmup)
        cache.check_status()
        # codes + bf16 scales (+ fp32 zero points for the 4-bit asymmetric cache) + q and out
        per_tok = 2 * 128 + 2 * 2 if args.bits == 8 else 2 * 64 + 2 * 2 + 2 * 4
        by = B * n_kv * ctx * per_tok + 2 * B * n_q * 128 * 2
        gbs = by / (ms * 1e-3) / 1e9
        emit("decode_attention_GBps", "GB/s", gbs, ms,
             {"workload": f"int{args.bits} decode attention", "streams": B, "q_heads": n_q, "kv_heads": n_kv, "context": ctx,
              "l2": "cache far larger than L2", "context_tokens_per_s": B * ctx / (ms * 1e-3)},
             {"bound": "hbm", "kernel": f"decode_attn_q{args.bits}_kernel", "achieved": gbs, "peak": peak, "peak_source": peak_src,
              "unit": "GB/s", "frac": gbs / peak, "traffic": None, "bytes": by}, launches)
        # budgeted step: H2O keeps 2048 tokens (256 recent + 1792 heavy) per (stream, KV head)
        acc = torch.rand(B * n_kv, ctx, device=dev)
        ts = torch.arange(ctx, dtype=torch.float32, device=dev).repeat(B * n_kv, 1)
        acc[:, ctx - 256:] = 0.0        # the recent window holds no heavy hitter: every segment keeps exactly 2048
        ms_sel = timed(lambda: ops.h2o_select(acc, ts, 1792, 256, as_bool=False), steps)
        by_sel = 2 * 4 * ctx * B * n_kv + B * n_kv * (ctx + 2048 * 4)
        emit("h2o_select_GBps", "GB/s", by_sel / (ms_sel * 1e-3) / 1e9, ms_sel,
             {"workload": "H2O segmented top-k", "segments": B * n_kv, "length": ctx, "heavy": 1792, "recent": 256},
             {"bound": "hbm", "kernel": "h2o_select_stream_kernel", "achieved": by_sel / (ms_sel * 1e-3) / 1e9, "peak": peak,
              "peak_source": peak_src, "unit": "GB/s", "frac": by_sel / (ms_sel * 1e-3) / 1e9 / peak, "traffic": None}, steps)
        # compaction of the kept rows (codes, scales, scores) and the decode step over the 2048-token budget
        if args.bits == 8 and ctx >= 2048:
            _, keep, cnt = ops.h2o_select(acc, ts, 1792, 256, as_bool=False)
            dst = pikv_b200.PagedKVCache(B, ctx, n_kv, device=dev)
            dacc, dts = torch.zeros_like(acc), torch.zeros_like(ts)
            ms_c = timed(lambda: cache.compact_into(dst, keep, cnt, True, acc, ts, dacc, dts), steps)
            by_c = 2 * B * n_kv * 2048 * (2 * 128 + 2 * 2 + 4 + 4)
            emit("h2o_compact_GBps", "GB/s", by_c / (ms_c * 1e-3) / 1e9, ms_c,
                 {"workload": "H2O compaction", "segments": B * n_kv, "kept": 2048},
                 {"bound": "hbm", "kernel": "h2o_compact_kernel", "achieved": by_c / (ms_c * 1e-3) / 1e9, "peak": peak,
                  "peak_source": peak_src, "unit": "GB/s", "frac": by_c / (ms_c * 1e-3) / 1e9 / peak, "traffic": None}, steps)
            dst.length.fill_(2048)
            ms_b = timed(lambda: dst.decode_attention(q, splits=args.splits, max_ctx=2048), steps)
            by_b = B * n_kv * 2048 * per_tok + 2 * B * n_q * 128 * 2
            emit("decode_attention_budgeted_GBps", "GB/s", by_b / (ms_b * 1e-3) / 1e9, ms_b,
                 {"workload": "int8 decode attention over the H2O budget", "streams": B, "context": 2048},
                 {"bound": "hbm", "kernel": "decode_attn_kernel<8>", "achieved": by_b / (ms_b * 1e-3) / 1e9, "peak": peak,
                  "peak_source": peak_src, "unit": "GB/s", "frac": by_b / (ms_b * 1e-3) / 1e9 / peak, "traffic": None}, steps)
            cache.check_status()
            dst.check_status()
    elif args.workload == "lowrank":
        M, K = args.rows, 1024
        x = torch.randn(M, K, device=dev).bfloat16()
        for r in (64, 32, 16):
            w = torch.nn.init.orthogonal_(torch.empty(K, K))[:r].contiguous().to(dev).bfloat16()
            ms = timed(lambda: ops.lowrank_project(x, w, None, relu=True), steps)
            by = M * K * 2 + M * r * 2
            gbs, tf = by / (ms * 1e-3) / 1e9, 2.0 * M * K * r / (ms * 1e-3) / 1e12
            emit("lowrank_project_GBps", "GB/s", gbs, ms,
                 {"workload": "low-rank KV projection", "rows": M, "hidden": K, "rank": r},
                 {"bound": "hbm", "kernel": "lowrank_gemm_kernel", "achieved": gbs, "peak": peak, "peak_source": peak_src,
                  "unit": "GB/s", "frac": gbs / peak, "traffic": None, "TFLOPs": tf}, steps)
        assert pikv_b200.lib().pikv_lowrank_error_state() == 0
    elif args.workload == "gate_net":
        # the two-layer gate net with its tail (tensor-bound); --rows tokens (a small count for profiler captures)
        Tn, Hn, En = args.rows, WORKLOAD["hidden"], WORKLOAD["experts"]
        gx = torch.randn(Tn, Hn, device=dev).bfloat16()
        gw1 = (torch.randn(Hn, Hn, device=dev) / Hn ** 0.5).bfloat16()
        gb1 = torch.zeros(Hn, device=dev)
        gw2, gb2 = gate_weights(Hn, En, 7)
        gw2, gb2 = gw2.to(dev), gb2.to(dev)
        capn = int(Tn * WORKLOAD["capacity_factor"] * WORKLOAD["top_k"] / En)
        gout = ops.gate_mlp_fused(gx, gw1, gb1, gw2, gb2, top_k=2, capacity=capn)
        ms = timed(lambda: ops.gate_mlp_fused(gx, gw1, gb1, gw2, gb2, top_k=2, capacity=capn, out=gout), steps)
        assert pikv_b200.lib().pikv_gate_error_state() == 0
        flops = 2.0 * Tn * Hn * Hn + 2.0 * Tn * Hn * En
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                tf_peak = float(json.load(f)["bf16_tflops_sustained"])
        except Exception:
            tf_peak = 1400.0
        tf = flops / (ms * 1e-3) / 1e12
        emit("gate_net_TFLOPs", "TFLOP/s", tf, ms, {"workload": "gate net (two layers + tail)", "tokens": Tn, "hidden": Hn, "experts": En},
             {"bound": "tensor", "kernel": "gate_mlp_kernel", "achieved": tf, "peak": tf_peak, "peak_source": "measured (sustained bf16)",
              "unit": "TFLOP/s", "frac": tf / tf_peak, "traffic": None}, steps)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the host-side port timing (profiling runs)")
    ap.add_argument("--schedule", choices=("pipelined", "serial"), default="pipelined",
                    help="single GPU: gate of batch i+1 overlapped with the append of batch i, or strictly serial")
    ap.add_argument("--no-large", action="store_true", help="skip the 8x-token secondary measurement")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other kernels' sub-records (decode attention, H2O, low-rank, 4-bit append)")
    ap.add_argument("--no-sharded", action="store_true", help="skip the expert-sharded configuration (striped cache: prefill + decode step)")
    ap.add_argument("--multi-warmup-s", type=float, default=3.0,
                    help="multi-GPU: seconds of untimed steps before the timed regions (stated in the line as warmup_s)")
    ap.add_argument("--workload", default="append", choices=["append", "decode", "lowrank", "gate_net"],
                    help="append = the headline route+quantise+append step; the others print lines for the other kernels")
    ap.add_argument("--streams", type=int, default=64)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--bits", type=int, default=8, choices=[4, 8], help="cache code width: 8 = int8 symmetric, 4 = 4-bit asymmetric (append and decode workloads)")
    ap.add_argument("--rows", type=int, default=262144)
    ap.add_argument("--shard-mode", default="peer", choices=["peer", "a2a"],
                    help="multi-GPU: peer = append kernel stores into the owner's pages over NVLink; a2a = pack + NCCL all_to_all")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload != "append":
        secondary_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
