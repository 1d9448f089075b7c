"""Striped expert-sharded KV cache: per-(expert, stream) caches whose rows rotate over the GPUs of one box.

The reference shards experts over ranks in contiguous blocks and sums the ranks' expert outputs with an
all_reduce (core/distributed/distributed_pikv.py:91-96, 174-194).  Here the unit is the cache of a pair
(expert, stream); its rows are cut into stripes that rotate over the ranks (striping.py), so the bytes of a
decode step spread evenly however skewed the routing is.  A stream's home rank gates its tokens, quantises
their K/V rows and stores each row straight into the owner's pages (pikv_kv_append_striped); a decode step is
pikv_shard_decode_post -> pikv_shard_decode_attn -> pikv_shard_decode_combine on every rank.  All of it runs
over peer-mapped memory (NVLink): no collective-library call, no multicast, every wait bounded.

One rank's state is a StripedShardedKVCache.  Its buffers come from one flat allocation per rank that every
rank has mapped: torch symmetric memory in a multi-process job (`StripedShardedKVCache.create`), or plain local
tensors when several ranks are emulated on one GPU for tests (`emulate_ranks`; their kernels then run one
after another on one stream, never concurrently).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np
import torch

from . import _lib, ops
from ._lib import check, lib
from .striping import StripedLayout, PAGE_TOKENS

_POOLS = ("k_codes", "v_codes", "k_scale", "v_scale")
_XCHG = ("q", "route", "post_flags", "part_o", "part_lse", "done_flags", "bar_flags")


def _region_sizes(layout: StripedLayout, num_pages: int, n_kv: int, n_q: int, top_k: int):
    L = lib()
    sizes = {"k_codes": num_pages * n_kv * PAGE_TOKENS * 128, "v_codes": num_pages * n_kv * PAGE_TOKENS * 128,
             "k_scale": num_pages * n_kv * PAGE_TOKENS * 2, "v_scale": num_pages * n_kv * PAGE_TOKENS * 2}
    for i, name in enumerate(_XCHG[:6]):
        sizes[name] = int(L.pikv_shard_decode_buffer_bytes(i, layout.world, layout.num_streams, top_k, n_q))
    sizes["bar_flags"] = layout.world * 4
    offs, o = {}, 0
    for name in _POOLS + _XCHG:
        offs[name] = o
        o += (sizes[name] + 255) // 256 * 256
    return sizes, offs, o


class StripedShardedKVCache:
    """One rank of the striped cache.  `flat` is this rank's allocation, `peer_ptrs[r]` rank r's allocation as
    seen from this GPU (peer_ptrs[rank] == flat.data_ptr())."""

    def __init__(self, layout: StripedLayout, rank: int, n_kv: int, n_q: int, top_k: int, cap_by_expert, flat: torch.Tensor,
                 peer_ptrs: List[int], num_pages: int, table: np.ndarray, wait_limit_us: int = 0):
        self.layout, self.rank, self.world = layout, rank, layout.world
        self.n_kv, self.n_q, self.top_k = n_kv, n_q, top_k
        self.device = flat.device
        self.num_pages, self.max_pages = num_pages, table.shape[1]
        self.flat, self.peer_ptrs = flat, list(peer_ptrs)
        self.sizes, self.offs, total = _region_sizes(layout, num_pages, n_kv, n_q, top_k)
        if flat.numel() < total:
            raise ValueError("flat allocation too small")
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.page_table = torch.from_numpy(np.ascontiguousarray(table)).to(dev)
        self.expert_rot = torch.from_numpy(layout.perm.astype(np.int32)).to(dev)
        self.expert_cap = torch.from_numpy(np.asarray(cap_by_expert, np.int32)).to(dev)
        self.streams_per_rank = layout.num_streams // layout.world
        if self.streams_per_rank * layout.world != layout.num_streams:
            raise ValueError("the streams must split evenly over the ranks")
        self.pair_len = torch.zeros(self.streams_per_rank, layout.num_experts, **i32)   # lengths of this rank's streams' pairs
        self.status = torch.zeros(1, **i32)
        self.seq = torch.zeros(1, **i32)
        self.counters = torch.zeros(2, **i32)
        self.bar_seq = torch.zeros(1, **i32)
        n_req = layout.num_streams * top_k
        self.req_seq, self.req_len, self.req_q = (torch.zeros(n_req, **i32) for _ in range(3))
        self.workspace = torch.empty(lib().pikv_decode_attn_workspace_bytes(n_req, n_q, n_kv, 0, 0), dtype=torch.uint8, device=dev)
        self.wait_limit_us = int(wait_limit_us)
        # scales of rows stored on other GPUs wait here (same offsets as in the owner's pool) and cross the link 32
        # bytes at a time after the append, instead of as one 2-byte packet per row
        entries = num_pages * n_kv * PAGE_TOKENS
        self.mirror_k = torch.zeros(self.world, entries, dtype=torch.bfloat16, device=dev) if self.world > 1 else None
        self.mirror_v = torch.zeros(self.world, entries, dtype=torch.bfloat16, device=dev) if self.world > 1 else None
        self._ctx = self._make_ctx()
        self._dec = self._make_decode_params()
        bp = _lib.PeerBarrierParams()
        bp.world, bp.rank, bp.seq, bp.status, bp.wait_limit_us = self.world, rank, self.bar_seq.data_ptr(), self.status.data_ptr(), self.wait_limit_us
        for r in range(self.world):
            bp.peer_flags[r] = self._ptr("bar_flags", r)
        self._bar = bp

    # -- construction ----------------------------------------------------------------------------------
    @staticmethod
    def plan(layout: StripedLayout, cap_by_expert, n_kv: int, n_q: int, top_k: int):
        """(page table, pages per rank, bytes per rank) for the given per-expert row capacities."""
        table, num_pages = layout.page_table(cap_by_expert)
        _, _, total = _region_sizes(layout, num_pages, n_kv, n_q, top_k)
        return table, num_pages, total

    @classmethod
    def create(cls, layout: StripedLayout, n_kv: int, n_q: int, top_k: int, cap_by_expert, device, group=None,
               wait_limit_us: int = 0) -> "StripedShardedKVCache":
        """This process's rank of a multi-process job: the allocation lives in torch symmetric memory (no
        multicast object is created) and every rank maps every other rank's."""
        import os
        table, num_pages, total = cls.plan(layout, cap_by_expert, n_kv, n_q, top_k)
        if layout.world == 1:
            flat = torch.zeros(total, dtype=torch.uint8, device=device)
            return cls(layout, 0, n_kv, n_q, top_k, cap_by_expert, flat, [flat.data_ptr()], num_pages, table, wait_limit_us)
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        rank = dist.get_rank(group)
        if dist.get_world_size(group) != layout.world:
            raise ValueError("layout.world differs from the process group's size")
        import torch.distributed._symmetric_memory as symm
        flat = symm.empty(total, dtype=torch.uint8, device=device)
        flat.zero_()
        torch.cuda.synchronize(device)
        hdl = symm.rendezvous(flat, group)
        out = cls(layout, rank, n_kv, n_q, top_k, cap_by_expert, flat, [int(hdl.buffer_ptrs[r]) for r in range(layout.world)],
                  num_pages, table, wait_limit_us)
        out._hdl = hdl
        return out

    def _ptr(self, name: str, r: int) -> int:
        return self.peer_ptrs[r] + self.offs[name]

    def _view(self, name: str, dtype, shape):
        o = self.offs[name]
        return self.flat[o:o + self.sizes[name]].view(dtype).view(shape)

    def _make_ctx(self):
        c = _lib.ShardDecodeCtx()
        lay = self.layout
        c.world, c.rank, c.num_experts, c.num_streams = self.world, self.rank, lay.num_experts, lay.num_streams
        c.top_k, c.n_q, c.stripe, c.streams_per_rank = self.top_k, self.n_q, lay.stripe, self.streams_per_rank
        c.expert_rot = self.expert_rot.data_ptr()
        for r in range(self.world):
            c.peer_q[r], c.peer_route[r], c.peer_post_flags[r] = self._ptr("q", r), self._ptr("route", r), self._ptr("post_flags", r)
            c.peer_part_o[r], c.peer_part_lse[r], c.peer_done_flags[r] = self._ptr("part_o", r), self._ptr("part_lse", r), self._ptr("done_flags", r)
        c.seq, c.counters, c.status, c.wait_limit_us = self.seq.data_ptr(), self.counters.data_ptr(), self.status.data_ptr(), self.wait_limit_us
        return c

    def _make_decode_params(self):
        p = _lib.DecodeParams()
        p.n_q, p.n_kv = self.n_q, self.n_kv
        p.page_table, p.num_seqs, p.max_pages, p.num_pages = self.page_table.data_ptr(), self.layout.num_pairs, self.max_pages, self.num_pages
        p.k_codes, p.v_codes = self._ptr("k_codes", self.rank), self._ptr("v_codes", self.rank)
        p.k_scale, p.v_scale = self._ptr("k_scale", self.rank), self._ptr("v_scale", self.rank)
        p.workspace, p.workspace_bytes, p.status = self.workspace.data_ptr(), self.workspace.numel(), self.status.data_ptr()
        return p

    # -- local pools as tensors (tests, checkpoints) -----------------------------------------------------
    def pool(self, name: str) -> torch.Tensor:
        if name.endswith("codes"):
            return self._view(name, torch.uint8, (self.num_pages, self.n_kv, PAGE_TOKENS, 128))
        return self._view(name, torch.bfloat16, (self.num_pages, self.n_kv, PAGE_TOKENS))

    def gather(self, seq: torch.Tensor, local_pos: torch.Tensor, which: str = "k", codes: bool = False):
        """Rows this rank holds, dequantised [n, n_kv*128] fp32 (and int8 codes): seq = pair ids, local_pos = slots
        on this rank (striping.StripedLayout.local_slot)."""
        seq, local_pos = ops._req(seq, "seq", torch.int32), ops._req(local_pos, "local_pos", torch.int32)
        n = seq.numel()
        out = torch.empty(n, self.n_kv * 128, dtype=torch.float32, device=self.device)
        cod = torch.empty(n, self.n_kv * 128, dtype=torch.int8, device=self.device) if codes else None
        check(lib().pikv_cache_gather(seq.data_ptr(), local_pos.data_ptr(), n, self.page_table.data_ptr(), self.layout.num_pairs,
                                      self.max_pages, self.num_pages, self.n_kv, 8, self._ptr(f"{which}_codes", self.rank),
                                      self._ptr(f"{which}_scale", self.rank), None, out.data_ptr(),
                                      None if cod is None else cod.data_ptr(), self.status.data_ptr(), ops._stream()),
              "pikv_cache_gather")
        return (out, cod) if codes else out

    def local_stream(self, stream: int) -> int:
        sl = stream - self.rank * self.streams_per_rank
        if not 0 <= sl < self.streams_per_rank:
            raise ValueError(f"stream {stream} is not at home on rank {self.rank}")
        return sl

    # -- writes ----------------------------------------------------------------------------------------
    def append_params(self, k: torch.Tensor, v: torch.Tensor, expert: torch.Tensor, pos: torch.Tensor, stream: int,
                      token_stream: Optional[torch.Tensor] = None):
        """Argument block of pikv_kv_append_striped for rows k, v [T, n_kv*128] bf16 of `stream` (or of
        token_stream[t]) going to experts expert [T,k] at positions pos [T,k] of their pairs."""
        sp = _lib.AppendStripedParams()
        b = sp.base
        T = k.shape[0]
        b.k, b.v, b.dtype, b.T, b.n_kv, b.top_k = k.data_ptr(), v.data_ptr(), _lib.PIKV_BF16, T, self.n_kv, expert.shape[1]
        b.dst_seq, b.slot, b.page_table = expert.data_ptr(), pos.data_ptr(), self.page_table.data_ptr()
        b.num_seqs, b.max_pages, b.num_pages = self.layout.num_pairs, self.max_pages, self.num_pages
        b.bits, b.symmetric, b.status = 8, 1, self.status.data_ptr()
        sp.world, sp.rank, sp.stripe = self.world, self.rank, self.layout.stripe
        sp.num_experts, sp.num_streams, sp.stream, sp.which = self.layout.num_experts, self.layout.num_streams, int(stream), 0
        sp.token_stream = None if token_stream is None else token_stream.data_ptr()
        sp.pair_len, sp.expert_rot, sp.expert_cap = None, self.expert_rot.data_ptr(), self.expert_cap.data_ptr()
        for r in range(self.world):
            sp.peer_k_codes[r], sp.peer_v_codes[r] = self._ptr("k_codes", r), self._ptr("v_codes", r)
            sp.peer_k_scale[r], sp.peer_v_scale[r] = self._ptr("k_scale", r), self._ptr("v_scale", r)
        if self.mirror_k is not None and token_stream is None:
            sp.mirror_k_scale, sp.mirror_v_scale = self.mirror_k.data_ptr(), self.mirror_v.data_ptr()
        return sp

    def push_params(self, stream: int, len_before: torch.Tensor, len_after: torch.Tensor):
        pp = _lib.StripedPushParams()
        pp.len_before, pp.len_after = len_before.data_ptr(), len_after.data_ptr()
        pp.expert_rot, pp.expert_cap, pp.page_table = self.expert_rot.data_ptr(), self.expert_cap.data_ptr(), self.page_table.data_ptr()
        pp.world, pp.rank, pp.stripe = self.world, self.rank, self.layout.stripe
        pp.num_experts, pp.num_streams, pp.stream = self.layout.num_experts, self.layout.num_streams, int(stream)
        pp.n_kv, pp.max_pages, pp.num_pages = self.n_kv, self.max_pages, self.num_pages
        pp.mirror_k_scale, pp.mirror_v_scale = self.mirror_k.data_ptr(), self.mirror_v.data_ptr()
        for r in range(self.world):
            pp.peer_k_scale[r], pp.peer_v_scale[r] = self._ptr("k_scale", r), self._ptr("v_scale", r)
        return pp

    def route_append(self, stream: int, k: torch.Tensor, v: torch.Tensor, *, act=None, w2=None, b2=None, logits=None,
                     top_k: Optional[int] = None, out: Optional[ops.GateResult] = None) -> ops.GateResult:
        """Gate T tokens of one of this rank's streams (hidden states act [T,H] with the gate's last layer, or
        given logits [T,E]), quantise their K/V rows and store every row on the rank that owns its stripe.
        The gate counts rows per expert from the pair's current length, so `slot` is the row's position in its
        pair; rows at or past the expert's capacity are dropped and the lengths stop there."""
        sl = self.local_stream(stream)
        top_k = top_k or self.top_k
        base = self.pair_len[sl]
        g = ops.gate_fused(act, w2, b2, logits=logits, top_k=top_k, capacity=0, slot_base=base, out=out)
        k = ops._req(k, "k", torch.bfloat16)
        v = ops._req(v, "v", torch.bfloat16)
        sp = self.append_params(k, v, g.topk_idx, g.slot, stream)
        check(lib().pikv_kv_append_striped(C.byref(sp), ops._stream()), "pikv_kv_append_striped")
        if self.mirror_k is not None:
            pp = self.push_params(stream, base, g.new_len)
            check(lib().pikv_shard_push_scales_striped(C.byref(pp), ops._stream()), "pikv_shard_push_scales_striped")
        torch.minimum(g.new_len, self.expert_cap, out=base)          # the pair lengths of this stream after the step
        return g

    # -- decode ----------------------------------------------------------------------------------------
    def decode_post(self, q_local: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor) -> None:
        q_local = ops._req(q_local, "q_local", torch.bfloat16)
        self._held = (q_local, ops._req(topk_idx, "topk_idx", torch.int32), ops._req(topk_w, "topk_w", torch.float32))
        check(lib().pikv_shard_decode_post(C.byref(self._ctx), self._held[0].data_ptr(), self._held[1].data_ptr(),
                                           self._held[2].data_ptr(), self.pair_len.data_ptr(), ops._stream()), "pikv_shard_decode_post")

    def decode_attend(self) -> None:
        check(lib().pikv_shard_decode_attn(C.byref(self._ctx), C.byref(self._dec), self.req_seq.data_ptr(),
                                           self.req_len.data_ptr(), self.req_q.data_ptr(), ops._stream()), "pikv_shard_decode_attn")

    def decode_combine(self, out: Optional[torch.Tensor] = None, mode: int = 0, lse: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(self.streams_per_rank, self.n_q, 128, dtype=torch.bfloat16, device=self.device)
        check(lib().pikv_shard_decode_combine(C.byref(self._ctx), self._held[1].data_ptr(), self._held[2].data_ptr(),
                                              self.pair_len.data_ptr(), out.data_ptr(), None if lse is None else lse.data_ptr(),
                                              int(mode), ops._stream()), "pikv_shard_decode_combine")
        return out

    def decode_step(self, q_local: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, out=None, mode: int = 0):
        """One decode step for this rank's streams: q_local [streams_per_rank, n_q, 128] bf16, their top-k experts
        and weights.  Every rank of the job must call it once per step."""
        self.decode_post(q_local, topk_idx, topk_w)
        self.decode_attend()
        return self.decode_combine(out, mode)

    def barrier(self) -> None:
        check(lib().pikv_peer_barrier(C.byref(self._bar), ops._stream()), "pikv_peer_barrier")

    def check_status(self) -> None:
        s = int(self.status.item())
        if s:
            raise _lib.PikvError(f"striped cache status word = {s:#x} (see PIKV_ST_* in include/pikv_b200.h)")


def emulate_ranks(layout: StripedLayout, n_kv: int, n_q: int, top_k: int, cap_by_expert, device) -> List[StripedShardedKVCache]:
    """All ranks of `layout` on ONE GPU, their allocations plain local tensors: for tests of the arithmetic.  The
    caller runs each phase for every rank before the next phase (post for all, attend for all, combine for all), on
    one stream, so that no kernel ever waits for one that has not run."""
    table, num_pages, total = StripedShardedKVCache.plan(layout, cap_by_expert, n_kv, n_q, top_k)
    flats = [torch.zeros(total, dtype=torch.uint8, device=device) for _ in range(layout.world)]
    ptrs = [f.data_ptr() for f in flats]
    return [StripedShardedKVCache(layout, r, n_kv, n_q, top_k, cap_by_expert, flats[r], ptrs, num_pages, table,
                                  wait_limit_us=50000) for r in range(layout.world)]
