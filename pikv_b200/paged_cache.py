"""Paged, quantised KV store in HBM and the kernels that write and read it.

A *sequence* owns one row of the page table: an expert's cache (routed append),
a decode stream, or an (expert, stream) pair on an expert-sharded GPU.  Pages
hold 16 tokens.  Pools (indexed by physical page id):

    k_codes, v_codes  uint8 [pages, n_kv, 16, 128*bits/8]   (chunk-swizzled rows)
    k_scale, v_scale  bf16  [pages, n_kv, 16]
    k_zp, v_zp        fp32  [pages, n_kv, 16]                (asymmetric only)

The row placement follows CacheSchedulingManager.update_cache
(core/single/cache_scheduling.py:430-436: contiguous rows, truncation at
capacity); the arithmetic of the stored codes is QuantizedCompressor.
_quantize_tensor (core/single/module/pikv_compression.py:945-1012) per
(token, head) slice of 128 channels.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import AppendParams, CompactParams, DecodeParams, PikvError, check, lib
from .ops import _p, _req, _stream, _workspace, _dtype_code, PAGE_TOKENS, HEAD_DIM


class PagedKVCache(torch.nn.Module):
    """Page pools + page table + per-sequence lengths, all registered buffers
    (so state_dict() carries the cache)."""

    def __init__(self, num_seqs: int, capacity: int, n_kv: int, bits: int = 8, symmetric: bool = True,
                 device="cuda", num_pages: Optional[int] = None, identity_table: bool = True):
        super().__init__()
        if bits not in (4, 8):
            raise ValueError("bits must be 4 or 8")
        self.num_seqs, self.n_kv, self.bits, self.symmetric = num_seqs, n_kv, bits, bool(symmetric)
        self.max_pages = (capacity + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.capacity = capacity
        self.num_pages = num_pages if num_pages is not None else num_seqs * self.max_pages
        row = HEAD_DIM * bits // 8
        dev = torch.device(device)
        z = lambda *s, dtype: torch.zeros(*s, dtype=dtype, device=dev)
        self.register_buffer("k_codes", z(self.num_pages, n_kv, PAGE_TOKENS, row, dtype=torch.uint8))
        self.register_buffer("v_codes", z(self.num_pages, n_kv, PAGE_TOKENS, row, dtype=torch.uint8))
        self.register_buffer("k_scale", z(self.num_pages, n_kv, PAGE_TOKENS, dtype=torch.bfloat16))
        self.register_buffer("v_scale", z(self.num_pages, n_kv, PAGE_TOKENS, dtype=torch.bfloat16))
        if not self.symmetric:
            self.register_buffer("k_zp", z(self.num_pages, n_kv, PAGE_TOKENS, dtype=torch.float32))
            self.register_buffer("v_zp", z(self.num_pages, n_kv, PAGE_TOKENS, dtype=torch.float32))
        else:
            self.k_zp = self.v_zp = None
        if identity_table:
            if self.num_pages < num_seqs * self.max_pages:
                raise ValueError("identity page table needs num_seqs * max_pages pages")
            pt = torch.arange(num_seqs * self.max_pages, dtype=torch.int32, device=dev).view(num_seqs, self.max_pages)
        else:
            pt = torch.full((num_seqs, self.max_pages), -1, dtype=torch.int32, device=dev)
        self.register_buffer("page_table", pt)
        self.register_buffer("length", z(num_seqs, dtype=torch.int32))
        self.register_buffer("status", z(1, dtype=torch.int32))

    # -- serialisation ---------------------------------------------------------------
    # The reference's checkpoint keeps one mean vector per cache (core/single/pikv_moe.py:456-505): the rows are
    # lost.  Here the cache itself is the state: pages, scales, zero points, page table and lengths are registered
    # buffers, so state_dict() / load_state_dict() move it, and these two calls add the geometry a loader needs
    # to rebuild the object, plus any score buffers of an eviction policy the caller passes along.
    def save_checkpoint(self, path, scores: Optional[dict] = None) -> None:
        torch.save({"format": "pikv_b200.paged_cache.v1",
                    "geometry": {"num_seqs": self.num_seqs, "capacity": self.capacity, "n_kv": self.n_kv, "bits": self.bits,
                                 "symmetric": self.symmetric, "num_pages": self.num_pages},
                    "state_dict": self.state_dict(),
                    "scores": {k: v.detach().clone() for k, v in (scores or {}).items()}}, path)

    @classmethod
    def load_checkpoint(cls, path, device="cuda"):
        """Returns (cache, scores): the cache rebuilt on `device` with every page, scale and length of the saved one."""
        blob = torch.load(path, map_location=torch.device(device), weights_only=False)
        if blob.get("format") != "pikv_b200.paged_cache.v1":
            raise PikvError(f"{path}: not a paged-cache checkpoint")
        g = blob["geometry"]
        cache = cls(g["num_seqs"], g["capacity"], g["n_kv"], bits=g["bits"], symmetric=g["symmetric"], device=device,
                    num_pages=g["num_pages"], identity_table=False)
        cache.load_state_dict(blob["state_dict"])
        return cache, blob.get("scores", {})

    # -- writes --------------------------------------------------------------------
    def append(self, k: torch.Tensor, v: torch.Tensor, dst_seq: torch.Tensor, slot: torch.Tensor) -> None:
        """Quantise and store k, v [T, n_kv*128] at (dst_seq[t,j], slot[t,j]); slot < 0 is skipped.
        Does not touch `length` (the gate's new_len, or the caller, owns it)."""
        k = _req(k, "k")
        v = _req(v, "v", k.dtype)
        T = k.shape[0]
        if k.shape[1] != self.n_kv * HEAD_DIM or v.shape != k.shape:
            raise PikvError(f"k/v must be [T, {self.n_kv * HEAD_DIM}], got {tuple(k.shape)} / {tuple(v.shape)}")
        dst_seq = _req(dst_seq, "dst_seq", torch.int32)
        slot = _req(slot, "slot", torch.int32)
        if dst_seq.dim() == 1:
            dst_seq, slot = dst_seq[:, None], slot[:, None]
        p = AppendParams()
        p.k, p.v, p.dtype, p.T, p.n_kv, p.top_k = _p(k), _p(v), _dtype_code(k, "k"), T, self.n_kv, dst_seq.shape[1]
        p.dst_seq, p.slot, p.page_table = _p(dst_seq), _p(slot), _p(self.page_table)
        p.num_seqs, p.max_pages, p.num_pages = self.num_seqs, self.max_pages, self.num_pages
        p.bits, p.symmetric = self.bits, int(self.symmetric)
        p.k_codes, p.v_codes, p.k_scale, p.v_scale = _p(self.k_codes), _p(self.v_codes), _p(self.k_scale), _p(self.v_scale)
        p.k_zp, p.v_zp = _p(self.k_zp), _p(self.v_zp)
        p.status = _p(self.status)
        check(lib().pikv_kv_append_quant(C.byref(p), _stream()), "pikv_kv_append_quant")

    def append_rope(self, k: torch.Tensor, v: torch.Tensor, dst_seq: torch.Tensor, slot: torch.Tensor,
                    cos: torch.Tensor, sin: torch.Tensor, positions: Optional[torch.Tensor] = None) -> None:
        """append() with the rotary position embedding of core/single/pikv_attention.py:329-390 applied to K in
        registers before it is quantised (pikv_kv_append_rope).  cos, sin: [max_pos, 64] fp32 tables (the
        reference's cos_cached / sin_cached); positions [T] int32 (default: the token index).  bf16 K/V, int8
        symmetric cache."""
        if self.bits != 8 or not self.symmetric:
            raise PikvError("append_rope writes int8 symmetric caches")
        k = _req(k, "k", torch.bfloat16)
        v = _req(v, "v", torch.bfloat16)
        cos, sin = _req(cos, "cos", torch.float32), _req(sin, "sin", torch.float32)
        if cos.dim() != 2 or cos.shape[1] != HEAD_DIM // 2 or sin.shape != cos.shape:
            raise PikvError(f"cos / sin must be [max_pos, {HEAD_DIM // 2}]")
        T = k.shape[0]
        if k.shape[1] != self.n_kv * HEAD_DIM or v.shape != k.shape:
            raise PikvError(f"k/v must be [T, {self.n_kv * HEAD_DIM}]")
        dst_seq = _req(dst_seq, "dst_seq", torch.int32)
        slot = _req(slot, "slot", torch.int32)
        if dst_seq.dim() == 1:
            dst_seq, slot = dst_seq[:, None], slot[:, None]
        if positions is not None:
            positions = _req(positions, "positions", torch.int32)
        p = AppendParams()
        p.k, p.v, p.dtype, p.T, p.n_kv, p.top_k = _p(k), _p(v), _lib.PIKV_BF16, T, self.n_kv, dst_seq.shape[1]
        p.dst_seq, p.slot, p.page_table = _p(dst_seq), _p(slot), _p(self.page_table)
        p.num_seqs, p.max_pages, p.num_pages = self.num_seqs, self.max_pages, self.num_pages
        p.bits, p.symmetric = 8, 1
        p.k_codes, p.v_codes, p.k_scale, p.v_scale = _p(self.k_codes), _p(self.v_codes), _p(self.k_scale), _p(self.v_scale)
        p.status = _p(self.status)
        check(lib().pikv_kv_append_rope(C.byref(p), _p(cos), _p(sin), _p(positions), cos.shape[0], _stream()), "pikv_kv_append_rope")

    def _route_params(self, act, w2, b2, k, v, top_k, capacity, out, slot_base, want_probs):
        from . import ops
        act = _req(act, "act")
        w2 = _req(w2, "w2", act.dtype)
        k = _req(k, "k")
        v = _req(v, "v", k.dtype)
        T, H = act.shape
        E = w2.shape[0]
        if E != self.num_seqs:
            raise PikvError(f"the cache has {self.num_seqs} sequences, the gate {E} experts")
        cap = self.capacity if capacity is None else capacity
        dev = act.device
        if out is None:
            f32, i32 = dict(dtype=torch.float32, device=dev), dict(dtype=torch.int32, device=dev)
            out = ops.GateResult(probs=torch.empty(T, E, **f32) if want_probs else None,
                                 topk_idx=torch.empty(T, top_k, **i32), topk_w=torch.empty(T, top_k, **f32),
                                 slot=torch.empty(T, top_k, **i32), counts_k=torch.empty(top_k, E, **i32),
                                 prob_sum=torch.empty(E, **f32), new_len=torch.empty(E, **i32))
        need = lib().pikv_gate_workspace_bytes(T, E, top_k)
        if out.workspace is None or out.workspace.numel() < need:
            # owned by the result, so calls on different streams never share gate scratch
            out.workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        b2f = None if b2 is None else _req(b2.to(torch.float32), "b2", torch.float32)
        gp = _lib.GateParams()
        gp.act, gp.w2, gp.b2, gp.dtype = _p(act), _p(w2), _p(b2f), _dtype_code(act, "act")
        gp.T, gp.H, gp.E, gp.top_k, gp.temperature, gp.capacity = T, H, E, top_k, 1.0, int(cap)
        if slot_base is not None:
            slot_base = _req(slot_base, "slot_base", torch.int32)
        gp.slot_base = _p(slot_base)
        gp.probs, gp.topk_idx, gp.topk_w, gp.slot = _p(out.probs), _p(out.topk_idx), _p(out.topk_w), _p(out.slot)
        gp.counts_k, gp.prob_sum, gp.new_len = _p(out.counts_k), _p(out.prob_sum), _p(out.new_len)
        gp.workspace, gp.workspace_bytes = _p(out.workspace), out.workspace.numel()
        ap = AppendParams()
        ap.k, ap.v, ap.dtype, ap.T, ap.n_kv, ap.top_k = _p(k), _p(v), _dtype_code(k, "k"), T, self.n_kv, top_k
        ap.page_table = _p(self.page_table)
        ap.num_seqs, ap.max_pages, ap.num_pages = self.num_seqs, self.max_pages, self.num_pages
        ap.bits, ap.symmetric = self.bits, int(self.symmetric)
        ap.k_codes, ap.v_codes, ap.k_scale, ap.v_scale = _p(self.k_codes), _p(self.v_codes), _p(self.k_scale), _p(self.v_scale)
        ap.k_zp, ap.v_zp, ap.status = _p(self.k_zp), _p(self.v_zp), _p(self.status)
        return gp, ap, out, (act, w2, b2f, k, v, slot_base)

    def route_append(self, act: torch.Tensor, w2: torch.Tensor, b2: Optional[torch.Tensor], k: torch.Tensor,
                     v: torch.Tensor, top_k: int = 2, capacity: Optional[int] = None,
                     out: Optional["ops.GateResult"] = None, slot_base: Optional[torch.Tensor] = None,
                     want_probs: bool = True):
        """Gate the tokens and append their quantised K/V rows in one call (pikv_route_append): the
        same results as ops.gate_fused followed by append(), with the slot finalisation folded into the
        append kernel.  Sequences are the experts.  Returns the gate result."""
        gp, ap, out, keep = self._route_params(act, w2, b2, k, v, top_k, capacity, out, slot_base, want_probs)
        check(lib().pikv_route_append(C.byref(gp), C.byref(ap), _stream()), "pikv_route_append")
        return out

    # -- reads ---------------------------------------------------------------------
    def gather(self, seq: torch.Tensor, pos: torch.Tensor, which: str = "k", codes: bool = False):
        """Dequantised rows [n, n_kv*128] fp32 (and int8 codes when codes=True) in logical order."""
        seq = _req(seq, "seq", torch.int32)
        pos = _req(pos, "pos", torch.int32)
        n = seq.numel()
        dev = seq.device
        out = torch.empty(n, self.n_kv * HEAD_DIM, dtype=torch.float32, device=dev)
        cod = torch.empty(n, self.n_kv * HEAD_DIM, dtype=torch.int8, device=dev) if codes else None
        pool, sc, zp = (self.k_codes, self.k_scale, self.k_zp) if which == "k" else (self.v_codes, self.v_scale, self.v_zp)
        check(lib().pikv_cache_gather(_p(seq), _p(pos), n, _p(self.page_table), self.num_seqs, self.max_pages,
                                      self.num_pages, self.n_kv, self.bits, _p(pool), _p(sc), _p(zp), _p(out), _p(cod),
                                      _p(self.status), _stream()), "pikv_cache_gather")
        return (out, cod) if codes else out

    def decode_attention(self, q: torch.Tensor, seq_ids: Optional[torch.Tensor] = None,
                         seq_len: Optional[torch.Tensor] = None, splits: int = 0, want_lse: bool = False,
                         scores: Optional[torch.Tensor] = None, max_ctx: Optional[int] = None):
        """softmax(q K^T / sqrt(128)) V over each stream's cached context; q [B, n_q, 128] bf16.  max_ctx: the
        longest context in the batch if the caller knows it (the split count is chosen from it without a host
        read of the lengths; default: the cache's capacity).  Reads
        int8 symmetric (pikv_decode_attn_q8) and 4-bit asymmetric (pikv_decode_attn_q4) caches."""
        q8 = self.bits == 8 and self.symmetric
        if not q8 and not (self.bits == 4 and not self.symmetric):
            raise PikvError("decode_attention reads int8 symmetric and 4-bit asymmetric caches")
        q = _req(q, "q", torch.bfloat16)
        B, n_q, d = q.shape
        if d != HEAD_DIM:
            raise PikvError(f"head dim must be {HEAD_DIM}")
        if seq_ids is not None:
            seq_ids = _req(seq_ids, "seq_ids", torch.int32)
        if seq_len is None:
            seq_len = self.length if seq_ids is None else self.length[seq_ids.long()]
        seq_len = _req(seq_len, "seq_len", torch.int32)
        dev = q.device
        out = torch.empty_like(q)
        lse = torch.empty(B, n_q, dtype=torch.float32, device=dev) if (want_lse or scores is not None) else None
        if splits <= 0:
            splits = lib().pikv_decode_attn_default_splits(B, self.n_kv, max_ctx or self.max_pages * PAGE_TOKENS)
        ws = _workspace(dev, lib().pikv_decode_attn_workspace_bytes(B, n_q, self.n_kv, self.capacity, splits), "dec")
        p = DecodeParams()
        p.q, p.out, p.B, p.n_q, p.n_kv = _p(q), _p(out), B, n_q, self.n_kv
        p.seq_ids, p.seq_len, p.page_table = _p(seq_ids), _p(seq_len), _p(self.page_table)
        p.num_seqs, p.max_pages, p.num_pages = self.num_seqs, self.max_pages, self.num_pages
        p.k_codes, p.v_codes, p.k_scale, p.v_scale = _p(self.k_codes), _p(self.v_codes), _p(self.k_scale), _p(self.v_scale)
        p.splits, p.lse = splits, _p(lse)
        p.scores, p.score_stride = _p(scores), (scores.shape[-1] if scores is not None else 0)
        p.workspace, p.workspace_bytes, p.status = _p(ws), ws.numel(), _p(self.status)
        if q8:
            check(lib().pikv_decode_attn_q8(C.byref(p), _stream()), "pikv_decode_attn_q8")
        else:
            p.k_zp, p.v_zp = _p(self.k_zp), _p(self.v_zp)
            check(lib().pikv_decode_attn_q4(C.byref(p), _stream()), "pikv_decode_attn_q4")
        return (out, lse) if (want_lse or scores is not None) else out

    def h2o_workspace(self, B: int, n_q: int, max_ctx: Optional[int] = None):
        """Scratch for decode_attention_h2o: f16 probabilities [B, n_q, ctx] and the step maxima [B, n_q, ctx/16]."""
        ctx = max_ctx or self.max_pages * PAGE_TOKENS
        dev = self.k_codes.device
        return (torch.empty(B, n_q, ctx, dtype=torch.float16, device=dev),
                torch.empty(B, n_q, (ctx + PAGE_TOKENS - 1) // PAGE_TOKENS, dtype=torch.float32, device=dev))

    def decode_attention_h2o(self, q: torch.Tensor, acc: torch.Tensor, workspace=None, seq_ids: Optional[torch.Tensor] = None,
                             seq_len: Optional[torch.Tensor] = None):
        """decode_attention plus the H2O update acc[b * n_kv + h, pos] += sum over the group's query heads of the
        attention probability (core/single/pikv_moe.py:241-245 column sums fed to
        core/single/cache_scheduling.py:69-73): the decode kernel leaves f16 probabilities relative to their softmax
        step, pikv_h2o_accumulate_probs normalises them with the final log-sum-exp.  int8 symmetric caches."""
        if self.bits != 8 or not self.symmetric:
            raise PikvError("decode_attention_h2o reads int8 symmetric caches")
        q = _req(q, "q", torch.bfloat16)
        acc = _req(acc, "acc", torch.float32)
        B, n_q, _ = q.shape
        if workspace is None:
            workspace = self.h2o_workspace(B, n_q)
        probs, step_max = workspace
        if seq_ids is not None:
            seq_ids = _req(seq_ids, "seq_ids", torch.int32)
        if seq_len is None:
            seq_len = self.length if seq_ids is None else self.length[seq_ids.long()]
        seq_len = _req(seq_len, "seq_len", torch.int32)
        dev = q.device
        out = torch.empty_like(q)
        lse = torch.empty(B, n_q, dtype=torch.float32, device=dev)
        ws = _workspace(dev, lib().pikv_decode_attn_workspace_bytes(B, n_q, self.n_kv, self.capacity, 0), "dec")
        p = DecodeParams()
        p.q, p.out, p.B, p.n_q, p.n_kv = _p(q), _p(out), B, n_q, self.n_kv
        p.seq_ids, p.seq_len, p.page_table = _p(seq_ids), _p(seq_len), _p(self.page_table)
        p.num_seqs, p.max_pages, p.num_pages = self.num_seqs, self.max_pages, self.num_pages
        p.k_codes, p.v_codes, p.k_scale, p.v_scale = _p(self.k_codes), _p(self.v_codes), _p(self.k_scale), _p(self.v_scale)
        p.lse, p.workspace, p.workspace_bytes, p.status = _p(lse), _p(ws), ws.numel(), _p(self.status)
        p.probs16, p.step_max, p.probs_stride, p.step_stride = _p(probs), _p(step_max), probs.shape[-1], step_max.shape[-1]
        check(lib().pikv_decode_attn_q8(C.byref(p), _stream()), "pikv_decode_attn_q8")
        check(lib().pikv_h2o_accumulate_probs(_p(probs), probs.shape[-1], _p(step_max), step_max.shape[-1], _p(lse), _p(seq_len),
                                              B, n_q, self.n_kv, _p(acc), acc.shape[-1], _stream()), "pikv_h2o_accumulate_probs")
        return out

    # -- eviction ------------------------------------------------------------------
    def compact_into(self, dst: "PagedKVCache", keep_idx: torch.Tensor, kept_count: torch.Tensor, per_head: bool,
                     src_acc=None, src_ts=None, dst_acc=None, dst_ts=None) -> None:
        """Copy the kept rows (ascending original order) to positions 0.. of `dst`'s sequences."""
        keep_idx = _req(keep_idx, "keep_idx", torch.int32)
        kept_count = _req(kept_count, "kept_count", torch.int32)
        p = CompactParams()
        p.keep_idx, p.kept_count, p.keep_stride = _p(keep_idx), _p(kept_count), keep_idx.shape[1]
        p.num_seqs, p.n_kv, p.per_head, p.bits = self.num_seqs, self.n_kv, int(per_head), self.bits
        p.src_page_table, p.dst_page_table = _p(self.page_table), _p(dst.page_table)
        p.max_pages, p.num_pages = min(self.max_pages, dst.max_pages), min(self.num_pages, dst.num_pages)
        if self.max_pages != dst.max_pages:
            raise PikvError("compact_into: source and destination must share the page-table width")
        p.src_k_codes, p.src_v_codes, p.src_k_scale, p.src_v_scale = _p(self.k_codes), _p(self.v_codes), _p(self.k_scale), _p(self.v_scale)
        p.src_k_zp, p.src_v_zp = _p(self.k_zp), _p(self.v_zp)
        p.dst_k_codes, p.dst_v_codes, p.dst_k_scale, p.dst_v_scale = _p(dst.k_codes), _p(dst.v_codes), _p(dst.k_scale), _p(dst.v_scale)
        p.dst_k_zp, p.dst_v_zp = _p(dst.k_zp), _p(dst.v_zp)
        p.src_acc, p.src_ts, p.dst_acc, p.dst_ts = _p(src_acc), _p(src_ts), _p(dst_acc), _p(dst_ts)
        segments = self.num_seqs * (self.n_kv if per_head else 1)
        for name, src_t, dst_t in (("acc", src_acc, dst_acc), ("ts", src_ts, dst_ts)):
            if (src_t is None) != (dst_t is None):
                raise PikvError(f"compact_into: give src_{name} and dst_{name} together")
            if src_t is not None:
                _req(src_t, f"src_{name}", torch.float32), _req(dst_t, f"dst_{name}", torch.float32)
                if src_t.numel() != segments * src_t.shape[-1] or dst_t.numel() != segments * dst_t.shape[-1]:
                    raise PikvError(f"compact_into: src_{name} / dst_{name} must have one row per segment ({segments})")
                if dst_t.shape[-1] < keep_idx.shape[1]:
                    raise PikvError(f"compact_into: dst_{name} rows are shorter than keep_idx rows")
        if src_acc is not None and src_ts is not None and (src_acc.shape[-1] != src_ts.shape[-1] or dst_acc.shape[-1] != dst_ts.shape[-1]):
            raise PikvError("compact_into: scores and timestamps must share their row lengths")
        first_src, first_dst = (src_acc, dst_acc) if src_acc is not None else (src_ts, dst_ts)
        p.score_stride = first_src.shape[-1] if first_src is not None else 0
        p.dst_score_stride = first_dst.shape[-1] if first_dst is not None else 0
        p.status = _p(self.status)
        check(lib().pikv_h2o_compact(C.byref(p), _stream()), "pikv_h2o_compact")

    def unpack_records(self, recv_buf: torch.Tensor, n_records: int, seq_offset: int = 0,
                       seg_start: Optional[torch.Tensor] = None, seg_base: Optional[torch.Tensor] = None) -> None:
        """Store records received from the token all-to-all (see ops.a2a_pack) into the pages.  Record
        sequence ids are global: seq_offset is subtracted.  seg_start [S+1] / seg_base [S, num_seqs] add a
        per-(source segment, sequence) base to the record's slot; positions >= capacity are dropped."""
        if self.bits != 8 or not self.symmetric:
            raise PikvError("records carry int8 symmetric codes")
        recv_buf = _req(recv_buf, "recv_buf", torch.uint8)
        n_seg = 0
        if seg_start is not None:
            seg_start = _req(seg_start, "seg_start", torch.int32)
            seg_base = _req(seg_base, "seg_base", torch.int32)
            n_seg = seg_start.numel() - 1
        check(lib().pikv_a2a_unpack(_p(recv_buf), n_records, self.n_kv, _p(self.page_table), self.num_seqs,
                                    self.max_pages, self.num_pages, seq_offset, self.capacity, _p(seg_start), _p(seg_base),
                                    n_seg, _p(self.k_codes), _p(self.v_codes), _p(self.k_scale), _p(self.v_scale),
                                    _p(self.status), _stream()), "pikv_a2a_unpack")

    def check_status(self) -> None:
        """Raise if any kernel flagged a bad index, page or a wait that ran out (synchronises)."""
        s = int(self.status.item())
        if s:
            raise PikvError(f"cache status word = {s:#x} (see PIKV_ST_* in include/pikv_b200.h)")
