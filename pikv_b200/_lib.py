"""ctypes binding of libpikv_b200.so (the C ABI declared in include/pikv_b200.h).

The library is loaded lazily by `lib()`.  There is no fallback: if the shared
object is missing or does not load, `lib()` raises and every operator of this
package fails with that error.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libpikv_b200.so")

PIKV_F32, PIKV_BF16 = 0, 1
MASK_NONE, MASK_SINGLE, MASK_MODULE, MASK_BIAS = 0, 1, 2, 3
GATE_WHOLE, GATE_SCORE, GATE_SLOTS, GATE_FORCE_SIMT = 0, 1, 2, 0x100
ST_BAD_SEQ, ST_BAD_PAGE, ST_BAD_INDEX, ST_WAIT_TIMEOUT = 1, 2, 8, 16
PAGE_TOKENS = 16
HEAD_DIM = 128
ABI_VERSION = 1

vp, i32, f32, sz, u64 = C.c_void_p, C.c_int32, C.c_float, C.c_size_t, C.c_uint64


class PikvError(RuntimeError):
    """A pikv_* entry point returned a negative status."""


class GateParams(C.Structure):
    _fields_ = [
        ("act", vp), ("w2", vp), ("b2", vp), ("logits_in", vp),
        ("dtype", i32), ("T", i32), ("H", i32), ("E", i32), ("top_k", i32),
        ("expert_mask", vp), ("mask_mode", i32), ("correction", vp),
        ("temperature", f32), ("renorm_eps", f32), ("capacity", i32), ("slot_base", vp),
        ("probs", vp), ("topk_idx", vp), ("topk_w", vp), ("slot", vp), ("counts_k", vp),
        ("prob_sum", vp), ("new_len", vp), ("workspace", vp), ("workspace_bytes", sz), ("phase", i32),
    ]


class AppendParams(C.Structure):
    _fields_ = [
        ("k", vp), ("v", vp), ("dtype", i32), ("T", i32), ("n_kv", i32), ("top_k", i32),
        ("dst_seq", vp), ("slot", vp), ("page_table", vp),
        ("num_seqs", i32), ("max_pages", i32), ("num_pages", i32), ("bits", i32), ("symmetric", i32),
        ("k_codes", vp), ("v_codes", vp), ("k_scale", vp), ("v_scale", vp), ("k_zp", vp), ("v_zp", vp),
        ("status", vp),
    ]


class AppendShardedParams(C.Structure):
    _fields_ = [
        ("base", AppendParams), ("world", i32), ("seqs_per_rank", i32), ("capacity", i32), ("slot_base", vp),
        ("peer_k_codes", vp * 8), ("peer_v_codes", vp * 8), ("peer_k_scale", vp * 8), ("peer_v_scale", vp * 8),
        ("rank", i32), ("which", i32), ("mirror_k_scale", vp), ("mirror_v_scale", vp),
    ]


class ShardPushParams(C.Structure):
    _fields_ = [
        ("counts_k", vp), ("slot_base", vp), ("page_table", vp),
        ("top_k", i32), ("E", i32), ("world", i32), ("rank", i32), ("seqs_per_rank", i32), ("capacity", i32),
        ("n_kv", i32), ("max_pages", i32), ("num_pages", i32),
        ("mirror_k_scale", vp), ("mirror_v_scale", vp), ("peer_k_scale", vp * 8), ("peer_v_scale", vp * 8),
    ]


class ShardExchangeParams(C.Structure):
    _fields_ = [
        ("counts_k", vp), ("top_k", i32), ("E", i32), ("world", i32), ("rank", i32), ("capacity", i32),
        ("start_empty", i32), ("peer_gather", vp * 8), ("peer_flags", vp * 8), ("seq", vp), ("len_all", vp),
        ("slot_base", vp), ("status", vp), ("wait_limit_us", i32),
    ]


class AppendStripedParams(C.Structure):
    _fields_ = [
        ("base", AppendParams), ("world", i32), ("rank", i32), ("stripe", i32), ("num_experts", i32), ("num_streams", i32),
        ("stream", i32), ("which", i32), ("token_stream", vp), ("pair_len", vp), ("expert_rot", vp), ("expert_cap", vp),
        ("peer_k_codes", vp * 8), ("peer_v_codes", vp * 8), ("peer_k_scale", vp * 8), ("peer_v_scale", vp * 8),
        ("mirror_k_scale", vp), ("mirror_v_scale", vp),
    ]


class StripedPushParams(C.Structure):
    _fields_ = [
        ("len_before", vp), ("len_after", vp), ("expert_rot", vp), ("expert_cap", vp), ("page_table", vp),
        ("world", i32), ("rank", i32), ("stripe", i32), ("num_experts", i32), ("num_streams", i32), ("stream", i32),
        ("n_kv", i32), ("max_pages", i32), ("num_pages", i32),
        ("mirror_k_scale", vp), ("mirror_v_scale", vp), ("peer_k_scale", vp * 8), ("peer_v_scale", vp * 8),
    ]


class ShardDecodeCtx(C.Structure):
    _fields_ = [
        ("world", i32), ("rank", i32), ("num_experts", i32), ("num_streams", i32), ("top_k", i32), ("n_q", i32),
        ("stripe", i32), ("streams_per_rank", i32), ("expert_rot", vp),
        ("peer_q", vp * 8), ("peer_route", vp * 8), ("peer_post_flags", vp * 8), ("peer_part_o", vp * 8),
        ("peer_part_lse", vp * 8), ("peer_done_flags", vp * 8), ("seq", vp), ("counters", vp), ("status", vp),
        ("wait_limit_us", i32),
    ]


class PeerBarrierParams(C.Structure):
    _fields_ = [("world", i32), ("rank", i32), ("peer_flags", vp * 8), ("seq", vp), ("status", vp), ("wait_limit_us", i32)]


XCHG_RING = 4
XCHG_FAILED = 0x80000000


class CompactParams(C.Structure):
    _fields_ = [
        ("keep_idx", vp), ("kept_count", vp),
        ("keep_stride", i32), ("num_seqs", i32), ("n_kv", i32), ("per_head", i32), ("bits", i32),
        ("src_page_table", vp), ("dst_page_table", vp), ("max_pages", i32), ("num_pages", i32),
        ("src_k_codes", vp), ("src_v_codes", vp), ("src_k_scale", vp), ("src_v_scale", vp),
        ("src_k_zp", vp), ("src_v_zp", vp),
        ("dst_k_codes", vp), ("dst_v_codes", vp), ("dst_k_scale", vp), ("dst_v_scale", vp),
        ("dst_k_zp", vp), ("dst_v_zp", vp),
        ("src_acc", vp), ("src_ts", vp), ("dst_acc", vp), ("dst_ts", vp), ("score_stride", i32),
        ("dst_score_stride", i32), ("status", vp),
    ]


class DecodeParams(C.Structure):
    _fields_ = [
        ("q", vp), ("out", vp), ("B", i32), ("n_q", i32), ("n_kv", i32),
        ("seq_ids", vp), ("seq_len", vp), ("page_table", vp),
        ("num_seqs", i32), ("max_pages", i32), ("num_pages", i32),
        ("k_codes", vp), ("v_codes", vp), ("k_scale", vp), ("v_scale", vp),
        ("splits", i32), ("lse", vp), ("scores", vp), ("score_stride", i32),
        ("workspace", vp), ("workspace_bytes", sz), ("status", vp), ("k_zp", vp), ("v_zp", vp),
        ("probs16", vp), ("step_max", vp), ("probs_stride", i32), ("step_stride", i32),
    ]


# name -> (restype, argtypes); every symbol include/pikv_b200.h declares
SIGNATURES = {
    "pikv_abi_version": (i32, []),
    "pikv_last_error": (C.c_char_p, []),
    "pikv_launch_count": (u64, []),
    "pikv_gate_workspace_bytes": (sz, [i32, i32, i32]),
    "pikv_gate_fused": (i32, [C.POINTER(GateParams), vp]),
    "pikv_gate_error_state": (i32, []),
    "pikv_gate_mlp_fused": (i32, [C.POINTER(GateParams), vp, i32, vp, vp, vp]),
    "pikv_dispatch_scatter": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp]),
    "pikv_kv_append_quant": (i32, [C.POINTER(AppendParams), vp]),
    "pikv_kv_append_rope": (i32, [C.POINTER(AppendParams), vp, vp, vp, i32, vp]),
    "pikv_route_append": (i32, [C.POINTER(GateParams), C.POINTER(AppendParams), vp]),
    "pikv_kv_append_sharded": (i32, [C.POINTER(AppendShardedParams), vp]),
    "pikv_shard_plan": (i32, [vp, i32, i32, i32, i32, vp, vp, vp]),
    "pikv_shard_exchange_plan": (i32, [C.POINTER(ShardExchangeParams), vp]),
    "pikv_h2o_select_variant": (i32, [i32]),
    "pikv_peer_barrier": (i32, [C.POINTER(PeerBarrierParams), vp]),
    "pikv_kv_append_striped": (i32, [C.POINTER(AppendStripedParams), vp]),
    "pikv_shard_push_scales_striped": (i32, [C.POINTER(StripedPushParams), vp]),
    "pikv_shard_decode_buffer_bytes": (sz, [i32, i32, i32, i32, i32]),
    "pikv_shard_decode_post": (i32, [C.POINTER(ShardDecodeCtx), vp, vp, vp, vp, vp]),
    "pikv_shard_decode_attn": (i32, [C.POINTER(ShardDecodeCtx), C.POINTER(DecodeParams), vp, vp, vp, vp]),
    "pikv_shard_decode_combine": (i32, [C.POINTER(ShardDecodeCtx), vp, vp, vp, vp, vp, i32, vp]),
    "pikv_shard_push_scales": (i32, [C.POINTER(ShardPushParams), vp]),
    "pikv_cache_gather": (i32, [vp, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp]),
    "pikv_quant_block_workspace_bytes": (sz, [i32, i32, i32]),
    "pikv_quant_block": (i32, [vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, sz, vp]),
    "pikv_h2o_accumulate": (i32, [vp, vp, i32, vp, vp, i32, f32, f32, vp, vp]),
    "pikv_h2o_select": (i32, [vp, vp, i32, i32, vp, i32, i32, i32, vp, vp, i32, vp, vp]),
    "pikv_h2o_compact": (i32, [C.POINTER(CompactParams), vp]),
    "pikv_decode_attn_workspace_bytes": (sz, [i32, i32, i32, i32, i32]),
    "pikv_decode_attn_default_splits": (i32, [i32, i32, i32]),
    "pikv_decode_attn_q8": (i32, [C.POINTER(DecodeParams), vp]),
    "pikv_decode_attn_q4": (i32, [C.POINTER(DecodeParams), vp]),
    "pikv_decode_attn_static_scratch_bytes": (sz, []),
    "pikv_decode_attn_q8_static": (i32, [C.POINTER(DecodeParams), vp]),
    "pikv_h2o_accumulate_probs": (i32, [vp, i32, vp, i32, vp, vp, i32, i32, i32, vp, i32, vp]),
    "pikv_h2o_accumulate_attn": (i32, [vp, i32, vp, vp, i32, i32, i32, vp, i32, vp]),
    "pikv_lowrank_project": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]),
    "pikv_lowrank_error_state": (i32, []),
    "pikv_a2a_record_bytes": (sz, [i32]),
    "pikv_a2a_pack": (i32, [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp]),
    "pikv_a2a_unpack": (i32, [vp, i32, i32, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp, vp, vp, vp]),
}

_LIB = None


def lib() -> C.CDLL:
    """Load libpikv_b200.so once and type every entry point."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise PikvError(
            f"{LIB_PATH} not found: build it with `python -m pikv_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    handle = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)   # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    got = handle.pikv_abi_version()
    if got != ABI_VERSION:
        raise PikvError(f"libpikv_b200.so has ABI {got}, this package expects {ABI_VERSION}")
    _LIB = handle
    return _LIB


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().pikv_last_error().decode("utf-8", "replace")
        raise PikvError(f"{what} failed with status {rc}: {msg}")


def launch_count() -> int:
    return int(lib().pikv_launch_count())
