"""Expert-sharded routed KV cache: one process per GPU, token all-to-all over NCCL.

The reference's expert-parallel model replicates the router and every token on
every rank, lets each rank run its contiguous block of experts on all tokens and
sums the results with one all_reduce (core/distributed/distributed_pikv.py:91-96,
174-194).  Here tokens are data-parallel: every rank gates its own tokens, packs
the quantised K/V rows of each routed (token, expert) pair into fixed-size records
ordered by destination, and one all_to_all_single moves each record to the rank
that owns the expert (contiguous blocks, as in the reference), where it is stored
into that rank's paged cache.

Slot order on the owner is (source rank, token, k) lexicographic, which equals the
single-GPU order when the global batch is split contiguously over the ranks: the
N-GPU cache holds exactly the rows, codes and slots of the 1-GPU cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from . import ops
from .paged_cache import PagedKVCache


def experts_per_rank(num_experts: int, world: int) -> int:
    """Contiguous expert blocks, core/distributed/distributed_pikv.py:91-96."""
    if num_experts % world != 0:
        raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
    return num_experts // world


@dataclass
class ExchangePlan:
    send_splits: np.ndarray   # [world] records this rank sends to each rank
    recv_splits: np.ndarray   # [world] records this rank receives from each rank
    seq_prefix: np.ndarray    # [E] first record index of each expert in this rank's send buffer
    seg_start: np.ndarray     # [world+1] first received record of each source rank
    seg_base: np.ndarray      # [world, E_local] slot of the first record of (source, local expert)
    new_len: np.ndarray       # [E_local] lengths after the step
    n_send: int
    n_recv: int


def plan_exchange(counts_all: np.ndarray, rank: int, lengths: np.ndarray, capacity: int) -> ExchangePlan:
    """Everything the exchange needs, from the all-gathered per-rank expert counts.

    counts_all [world, E]: selections of expert e by the tokens of each rank (what the gate counts).
    lengths [E_local]: current length of this rank's experts.  Pure host arithmetic (numpy)."""
    counts_all = np.asarray(counts_all, np.int64)
    world, E = counts_all.shape
    per = experts_per_rank(E, world)
    mine = counts_all[rank]
    send_splits = mine.reshape(world, per).sum(1)
    lo, hi = rank * per, (rank + 1) * per
    recv_counts = counts_all[:, lo:hi]                       # [source, local expert]
    recv_splits = recv_counts.sum(1)
    seq_prefix = np.concatenate([[0], np.cumsum(mine)[:-1]])
    seg_start = np.concatenate([[0], np.cumsum(recv_splits)])
    seg_base = np.asarray(lengths, np.int64)[None, :] + np.cumsum(recv_counts, axis=0) - recv_counts
    new_len = np.minimum(np.asarray(lengths, np.int64) + recv_counts.sum(0), capacity)
    return ExchangePlan(send_splits.astype(np.int64), recv_splits.astype(np.int64), seq_prefix.astype(np.int32),
                        seg_start.astype(np.int32), seg_base.astype(np.int32), new_len.astype(np.int32),
                        int(send_splits.sum()), int(recv_splits.sum()))


class ExpertShardedKVCache:
    """This rank's slice of the routed cache plus the exchange that feeds it."""

    def __init__(self, num_experts: int, capacity: int, n_kv: int, device, group=None, max_records: int = 0):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.num_experts, self.n_kv, self.capacity = num_experts, n_kv, capacity
        self.per = experts_per_rank(num_experts, self.world)
        self.device = torch.device(device)
        self.cache = PagedKVCache(self.per, capacity, n_kv, device=self.device)
        self.rec = ops.a2a_record_bytes(n_kv)
        self._lengths = np.zeros(self.per, np.int64)
        self._send = self._recv = None
        self.max_records = max_records
        self.last_plan: Optional[ExchangePlan] = None

    def _buffers(self, n_send: int, n_recv: int):
        need_s, need_r = max(n_send, 1, self.max_records) * self.rec, max(n_recv, 1, self.max_records) * self.rec
        if self._send is None or self._send.numel() < need_s:
            self._send = torch.empty(need_s, dtype=torch.uint8, device=self.device)
        if self._recv is None or self._recv.numel() < need_r:
            self._recv = torch.empty(need_r, dtype=torch.uint8, device=self.device)
        return self._send, self._recv

    def route_append(self, act: torch.Tensor, w2: torch.Tensor, b2: Optional[torch.Tensor], k: torch.Tensor,
                     v: torch.Tensor, top_k: int = 2, out: Optional[ops.GateResult] = None) -> ops.GateResult:
        """Gate this rank's tokens, exchange the quantised rows, store what this rank owns."""
        g = ops.gate_fused(act, w2, b2, top_k=top_k, capacity=0, out=out)       # slot = rank inside (this rank, expert)
        counts = g.counts_k.sum(0).to(torch.int32)
        if self.world > 1:
            gathered = torch.empty(self.world, self.num_experts, dtype=torch.int32, device=self.device)
            dist.all_gather_into_tensor(gathered, counts, group=self.group)
        else:
            gathered = counts[None]
        plan = plan_exchange(gathered.cpu().numpy(), self.rank, self._lengths, self.capacity)   # one host read per step
        self.last_plan = plan
        send, recv = self._buffers(plan.n_send, plan.n_recv)
        to_dev = lambda a: torch.from_numpy(a).to(self.device, non_blocking=True)
        ops.a2a_pack(k, v, self.n_kv, g.topk_idx, g.slot, plan.n_send, seq_prefix=to_dev(plan.seq_prefix), out=send)
        if self.world > 1:
            dist.all_to_all_single(recv[: plan.n_recv * self.rec], send[: plan.n_send * self.rec],
                                   output_split_sizes=(plan.recv_splits * self.rec).tolist(),
                                   input_split_sizes=(plan.send_splits * self.rec).tolist(), group=self.group)
        else:
            recv = send
        self.cache.unpack_records(recv, plan.n_recv, seq_offset=self.rank * self.per,
                                  seg_start=to_dev(plan.seg_start), seg_base=to_dev(plan.seg_base.reshape(-1)))
        self._lengths = plan.new_len.astype(np.int64)
        self.cache.length.copy_(to_dev(plan.new_len))
        return g

    def reset(self):
        self._lengths[:] = 0
        self.cache.length.zero_()


class PeerShardedKVCache:
    """Expert-sharded cache whose append kernel stores straight into the owner GPU's pages.

    Every rank's page pools live in one symmetric-memory allocation, so each rank holds a
    peer-mapped pointer to every other rank's pools (NVLink, NVSwitch).  A step is: gate the local
    tokens -> one one-CTA kernel that exchanges the E selection counts with every rank through
    peer memory (stores + flags, bounded wait) and plans the step (slot of this rank's first row in
    every sequence, new lengths) -> the quantise + append kernel, whose stores for remote sequences
    cross NVLink as plain 16-byte stores -> (before anybody reads the rows) a symmetric-memory
    barrier.  The step is three of this library's kernels and no collective-library call; nothing
    touches the host, and no copy of a row is staged in HBM: per-GPU HBM traffic is that of the
    single-GPU step.  No multicast object is created (plain peer pointers only).
    """

    def __init__(self, num_experts: int, capacity: int, n_kv: int, device, group=None, wait_limit_us: int = 0):
        import ctypes as C
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        self._C, self._lib = C, _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("one box: at most 8 ranks")
        self.num_experts, self.n_kv, self.capacity = num_experts, n_kv, capacity
        self.per = experts_per_rank(num_experts, self.world)
        self.device = torch.device(device)
        # the local cache object gives the layout; its pools are then re-homed into symmetric memory
        self.cache = PagedKVCache(self.per, capacity, n_kv, device=self.device)
        names = ("k_codes", "v_codes", "k_scale", "v_scale")
        sizes = [getattr(self.cache, n).numel() * getattr(self.cache, n).element_size() for n in names]
        ring = _lib.XCHG_RING
        sizes += [ring * self.world * num_experts * 4, ring * self.world * 4]      # count exchange: gather, flags
        sizes += [self.world * 4]                                                  # barrier flags
        self.wait_limit_us = int(wait_limit_us)                                    # 0: the library's default (2 s)
        offs = np.concatenate([[0], np.cumsum([(b + 255) // 256 * 256 for b in sizes])])
        self._buf = symm.empty(int(offs[-1]), dtype=torch.uint8, device=self.device)
        self._buf.zero_()
        torch.cuda.synchronize(self.device)      # flags are zero on every rank before any peer can raise one
        self._hdl = symm.rendezvous(self._buf, self.group)
        self._peer = {n: [int(self._hdl.buffer_ptrs[r]) + int(offs[i]) for r in range(self.world)]
                      for i, n in enumerate(names)}
        self._peer_gather = [int(self._hdl.buffer_ptrs[r]) + int(offs[4]) for r in range(self.world)]
        self._peer_flags = [int(self._hdl.buffer_ptrs[r]) + int(offs[5]) for r in range(self.world)]
        self._peer_bar = [int(self._hdl.buffer_ptrs[r]) + int(offs[6]) for r in range(self.world)]
        self.seq = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.bar_seq = torch.zeros(1, dtype=torch.int32, device=self.device)
        bp = _lib.PeerBarrierParams()
        bp.world, bp.rank, bp.seq, bp.status = self.world, self.rank, ops._p(self.bar_seq), ops._p(self.cache.status)
        bp.wait_limit_us = self.wait_limit_us
        for r in range(self.world):
            bp.peer_flags[r] = self._peer_bar[r]
        self._bar_params = bp
        # scales of rows stored on other GPUs wait here (same offsets as in the owner's pool) and cross the
        # link 32 bytes at a time after the append, instead of as one 2-byte packet per row
        entries = self.cache.k_scale.numel()
        self.mirror_k = torch.zeros(self.world, entries, dtype=torch.bfloat16, device=self.device) if self.world > 1 else None
        self.mirror_v = torch.zeros(self.world, entries, dtype=torch.bfloat16, device=self.device) if self.world > 1 else None
        self._start_empty = False
        for i, n in enumerate(names):
            old = getattr(self.cache, n)
            view = self._buf[int(offs[i]): int(offs[i]) + sizes[i]].view(old.dtype).view(old.shape)
            setattr(self.cache, n, view)
        mp = self.cache.max_pages
        table = (torch.arange(num_experts, device=self.device) % self.per)[:, None] * mp + torch.arange(mp, device=self.device)
        self.global_table = table.to(torch.int32).contiguous()
        self.len_all = torch.zeros(num_experts, dtype=torch.int32, device=self.device)
        self.slot_base = torch.zeros(num_experts, dtype=torch.int32, device=self.device)
        self.gathered = torch.zeros(self.world, num_experts, dtype=torch.int32, device=self.device)
        self.counts = torch.zeros(num_experts, dtype=torch.int32, device=self.device)

    def prepare(self, act, w2, b2, k, v, top_k: int = 2, out: Optional[ops.GateResult] = None, split: bool = False):
        """Bind one set of buffers to a step and return `run()`: the argument blocks are built once, so a
        call of run() is four C-ABI calls (gate, count exchange + plan, append, scale push), plus the barrier
        when asked, and no host arithmetic.  The buffers must stay alive and in place while run() is used."""
        C, L = self._C, self._lib
        act, w2 = ops._req(act, "act", torch.bfloat16), ops._req(w2, "w2", torch.bfloat16)
        k, v = ops._req(k, "k", torch.bfloat16), ops._req(v, "v", torch.bfloat16)
        T, H = act.shape
        E = self.num_experts
        if out is None:
            out = ops.gate_fused(act, w2, b2, top_k=top_k, capacity=0)
        # gate scratch owned by this binding: several prepared steps (lanes, buffer sets) run concurrently on
        # different streams, and the scratch holds the per-CTA counts the slot finalisation reads
        ws = torch.empty(max(1, L.lib().pikv_gate_workspace_bytes(T, E, top_k)), dtype=torch.uint8, device=self.device)
        out.workspace = ws
        b2f = None if b2 is None else ops._req(b2.to(torch.float32), "b2", torch.float32)
        gp = L.GateParams()
        gp.act, gp.w2, gp.b2, gp.dtype = ops._p(act), ops._p(w2), ops._p(b2f), L.PIKV_BF16
        gp.T, gp.H, gp.E, gp.top_k, gp.temperature, gp.capacity = T, H, E, top_k, 1.0, 0
        gp.probs, gp.topk_idx, gp.topk_w, gp.slot = ops._p(out.probs), ops._p(out.topk_idx), ops._p(out.topk_w), ops._p(out.slot)
        gp.counts_k, gp.prob_sum, gp.new_len = ops._p(out.counts_k), ops._p(out.prob_sum), ops._p(out.new_len)
        gp.workspace, gp.workspace_bytes = ops._p(ws), ws.numel()
        sp = L.AppendShardedParams()
        b = sp.base
        b.k, b.v, b.dtype, b.T, b.n_kv, b.top_k = ops._p(k), ops._p(v), L.PIKV_BF16, T, self.n_kv, top_k
        b.dst_seq, b.slot, b.page_table = ops._p(out.topk_idx), ops._p(out.slot), ops._p(self.global_table)
        b.num_seqs, b.max_pages, b.num_pages = E, self.cache.max_pages, self.cache.num_pages
        b.bits, b.symmetric, b.status = 8, 1, ops._p(self.cache.status)
        sp.world, sp.seqs_per_rank, sp.capacity, sp.slot_base = self.world, self.per, self.capacity, ops._p(self.slot_base)
        for r in range(self.world):
            sp.peer_k_codes[r], sp.peer_v_codes[r] = self._peer["k_codes"][r], self._peer["v_codes"][r]
            sp.peer_k_scale[r], sp.peer_v_scale[r] = self._peer["k_scale"][r], self._peer["v_scale"][r]
        sp.rank, sp.which = self.rank, 0
        sp.mirror_k_scale, sp.mirror_v_scale = ops._p(self.mirror_k), ops._p(self.mirror_v)
        pp = L.ShardPushParams()
        pp.counts_k, pp.slot_base, pp.page_table = ops._p(out.counts_k), ops._p(self.slot_base), ops._p(self.global_table)
        pp.top_k, pp.E, pp.world, pp.rank, pp.seqs_per_rank, pp.capacity = top_k, E, self.world, self.rank, self.per, self.capacity
        pp.n_kv, pp.max_pages, pp.num_pages = self.n_kv, self.cache.max_pages, self.cache.num_pages
        pp.mirror_k_scale, pp.mirror_v_scale = ops._p(self.mirror_k), ops._p(self.mirror_v)
        for r in range(self.world):
            pp.peer_k_scale[r], pp.peer_v_scale[r] = self._peer["k_scale"][r], self._peer["v_scale"][r]
        sp_local = sp_remote = None
        if split and self.world > 1:
            # the rows of this rank's own sequences and the rows that cross NVLink as two launches on two
            # streams: remote stores back up when the link is the bottleneck, and a launch that also holds
            # local rows would stall those behind them
            sp_local, sp_remote = type(sp).from_buffer_copy(sp), type(sp).from_buffer_copy(sp)
            sp_local.which, sp_remote.which = 1, 2
            side = torch.cuda.Stream(device=self.device)
        xp = L.ShardExchangeParams()
        xp.counts_k, xp.top_k, xp.E, xp.world, xp.rank, xp.capacity = ops._p(out.counts_k), top_k, E, self.world, self.rank, self.capacity
        for r in range(self.world):
            xp.peer_gather[r], xp.peer_flags[r] = self._peer_gather[r], self._peer_flags[r]
        xp.seq, xp.len_all, xp.slot_base, xp.status = ops._p(self.seq), ops._p(self.len_all), ops._p(self.slot_base), ops._p(self.cache.status)
        xp.wait_limit_us = self.wait_limit_us
        lib, keep = L.lib(), (act, w2, b2f, k, v, out, ws)

        def run(sync: bool = True):
            st = ops._stream()
            L.check(lib.pikv_gate_fused(C.byref(gp), st), "pikv_gate_fused")
            xp.start_empty, self._start_empty = int(self._start_empty), False
            L.check(lib.pikv_shard_exchange_plan(C.byref(xp), st), "pikv_shard_exchange_plan")
            if sp_local is None:
                L.check(lib.pikv_kv_append_sharded(C.byref(sp), st), "pikv_kv_append_sharded")
            else:
                cur = torch.cuda.current_stream()
                side.wait_stream(cur)
                with torch.cuda.stream(side):
                    L.check(lib.pikv_kv_append_sharded(C.byref(sp_remote), ops._stream()), "pikv_kv_append_sharded")
                L.check(lib.pikv_kv_append_sharded(C.byref(sp_local), st), "pikv_kv_append_sharded")
                cur.wait_stream(side)
            if self.world > 1:
                L.check(lib.pikv_shard_push_scales(C.byref(pp), st), "pikv_shard_push_scales")
            if sync:
                self.barrier()
            return out

        run._keep = keep
        return run

    def route_append(self, act, w2, b2, k, v, top_k: int = 2, out: Optional[ops.GateResult] = None,
                     sync: bool = True, split: bool = False) -> ops.GateResult:
        g = self.prepare(act, w2, b2, k, v, top_k, out, split)(sync)
        self.sync_lengths()
        return g

    def sync_lengths(self):
        """Copy this rank's slice of the replicated length table into the local cache object."""
        lo = self.rank * self.per
        self.cache.length.copy_(self.len_all[lo: lo + self.per])

    def barrier(self):
        """All ranks' append kernels are complete (and their remote stores visible) after this point
        of the stream: pikv_peer_barrier over flag words in the symmetric buffer, no host sync.  Like every
        wait of the library it is bounded: if a rank never arrives, PIKV_ST_WAIT_TIMEOUT is raised in the
        cache's status word and the stream carries on."""
        self._lib.check(self._lib.lib().pikv_peer_barrier(self._C.byref(self._bar_params), ops._stream()), "pikv_peer_barrier")

    def reset(self):
        """Empty the cache: the next step plans from zero lengths (no kernel is enqueued for this)."""
        self._start_empty = True


def make_bench_step(dev, rank, world, cfg, w2, b2, synth_inputs, mode: str = "peer"):
    """The benchmark step at `world` GPUs: every rank routes its own batch of cfg['tokens'] tokens
    (weak scaling) into the expert-sharded cache.  mode "peer": the append kernel stores into the
    owner GPU's pages over NVLink; mode "a2a": pack -> NCCL all_to_all -> unpack.  The cache is
    emptied every step so that steps are identical."""
    T, H, E, k = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["top_k"]
    n_kv = cfg["kv_heads"]
    kv = n_kv * cfg["head_dim"]
    cap = int(T * world * cfg["capacity_factor"] * k / E)
    import os
    R = int(os.environ.get("PIKV_BENCH_LANES", "6")) if mode == "peer" else 2
    sets = [synth_inputs(T, H, E, kv, 1000 * rank + i, device=dev) for i in range(R)]
    outs = [ops.gate_fused(sets[0][0], w2, b2, top_k=k, capacity=0) for _ in range(R)]
    hooks = {"begin": lambda: None, "end": lambda: None}
    if mode == "peer":
        # several steps in flight (six by default), one stream each, each with its own cache instance (own pools, own exchange
        # ring): the gate of one step overlaps the count exchange and the NVLink stores of the previous
        # one.  Nobody reads rows between the appends, so the cross-GPU barrier runs once, at the end.
        import os
        lanes = int(os.environ.get("PIKV_BENCH_LANES", "6"))
        shards = [PeerShardedKVCache(E, cap, n_kv, dev) for _ in range(lanes)]
        streams = [torch.cuda.Stream(device=dev) for _ in range(lanes)]
        how = f"append kernel stores into the owner GPU's pages over NVLink (peer pointers); {lanes} steps in flight"
        split = os.environ.get("PIKV_BENCH_SPLIT", "0") == "1"      # local and remote rows as two launches on two streams
        runs = [[shards[l].prepare(sets[i][0], w2, b2, sets[i][1], sets[i][2], top_k=k, out=outs[i], split=split)
                 for i in range(R)] for l in range(lanes)]

        import os
        graphs, launches_per_step = None, None
        if os.environ.get("PIKV_BENCH_MULTI_EAGER", "0") != "1":
            # a lane's step is four kernels of this library and nothing else (no collective-library call, no
            # host read), so it is captured once per (lane, buffer set) and replayed: one launch per step.
            # Every rank runs and captures in the same order (the count exchange numbers its steps).
            for lane in range(lanes):
                for i in range(R):
                    with torch.cuda.stream(streams[lane]):
                        shards[lane].reset()
                        runs[lane][i](sync=False)
            torch.cuda.synchronize()
            dist.barrier()
            graphs = [[None] * R for _ in range(lanes)]
            from . import _lib
            n0 = _lib.launch_count()
            for lane in range(lanes):
                for i in range(R):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=streams[lane]):
                        shards[lane].reset()
                        runs[lane][i](sync=False)
                    graphs[lane][i] = g
            launches_per_step = (_lib.launch_count() - n0) // (lanes * R)
            # (one graph per lane step, not one graph for several lanes: the lanes' exchange kernels wait for
            # their peers, and the parallel branches of a single graph did not run concurrently on every
            # rank, so such a graph ran into the bounded waits)
            how += "; each lane's step replayed as one CUDA graph"

        def step(i):
            lane = i % lanes
            with torch.cuda.stream(streams[lane]):
                if graphs is not None:
                    graphs[lane][i % R].replay()
                else:
                    shards[lane].reset()
                    runs[lane][i % R](sync=False)

        def begin():
            for st in streams:
                st.wait_stream(torch.cuda.current_stream())

        def end():
            for shard, st in zip(shards, streams):
                with torch.cuda.stream(st):
                    shard.barrier()
                torch.cuda.current_stream().wait_stream(st)

        hooks = {"begin": begin, "end": end}

        def verify():
            """Outside the timing: one more step of buffer set 0 on every lane, then every lane's status word
            must be clear and its replicated lengths must equal the sum over the ranks of the selection counts
            (cut at the capacity)."""
            counts = outs[0].counts_k.sum(0).to(torch.int32)
            for lane in range(lanes):
                with torch.cuda.stream(streams[lane]):
                    shards[lane].reset()
                    runs[lane][0](sync=True)
            torch.cuda.synchronize()
            allc = torch.empty(world, E, dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(allc, counts)
            want = torch.clamp(allc.sum(0), max=cap).to(torch.int32)
            for lane in range(lanes):
                shards[lane].cache.check_status()
                if not torch.equal(shards[lane].len_all, want):
                    raise RuntimeError(f"lane {lane}: replicated lengths differ from the all-gathered counts")
            return lanes

        # bytes this rank's rows put on the link per step: int8 K + V codes and their bf16 scales, for the
        # (token, expert) pairs whose expert lives on another GPU (buffer set 0, measured from the gate's counts)
        c0 = outs[0].counts_k.sum(0)
        per = E // world
        remote = int(c0.sum().item() - c0[rank * per:(rank + 1) * per].sum().item())
        link_bytes = remote * (2 * kv + 2 * n_kv * 2)

        # end to end: the step's inputs come from pinned host memory and its routing result goes back, on
        # the lane's stream, every step
        h_sets = [tuple(x.cpu().pin_memory() for x in sets[i]) for i in range(R)]
        h_outs = [tuple(torch.empty_like(x, device="cpu").pin_memory()
                        for x in (outs[i].topk_idx, outs[i].topk_w, outs[i].slot, outs[i].new_len)) for i in range(R)]

        def e2e_step(i):
            lane = i % lanes
            with torch.cuda.stream(streams[lane]):
                for dst, src in zip(sets[i % R], h_sets[i % R]):
                    dst.copy_(src, non_blocking=True)
            step(i)
            with torch.cuda.stream(streams[lane]):
                o = outs[i % R]
                for dst, src in zip(h_outs[i % R], (o.topk_idx, o.topk_w, o.slot, o.new_len)):
                    dst.copy_(src, non_blocking=True)

        e2e_io = (e2e_step, sum(x.numel() * x.element_size() for x in h_sets[0]),
                  sum(x.numel() * x.element_size() for x in h_outs[0]))
    else:
        e2e_io = None
        shard = ExpertShardedKVCache(E, cap, n_kv, dev, max_records=int(T * k * 1.5))
        how = "pack -> NCCL all_to_all -> unpack"

        def step(i):
            act, K, V = sets[i % R]
            shard.reset()
            shard.route_append(act, w2, b2, K, V, top_k=k, out=outs[i % R])

    extra = {"parallelism": f"tokens data-parallel, {E} experts sharded {E // world} per GPU; {how}",
             "buffer_sets": R, "hooks": hooks}
    if mode == "peer":
        extra["verify"] = verify
        extra["link_bytes_per_step"] = link_bytes
    if mode == "peer" and launches_per_step is not None:
        extra["launches_per_step"] = launches_per_step
    if e2e_io is not None:
        extra["e2e_io"] = e2e_io
    return step, extra
