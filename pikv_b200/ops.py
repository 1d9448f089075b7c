"""Functional wrappers: torch CUDA tensors in, kernels launched through the C ABI.

Every function enqueues on the current torch CUDA stream and returns torch
tensors it allocated.  Inputs are borrowed and never modified unless the
docstring says so.  Nothing here computes on the CPU: a tensor that is not on
a CUDA device is an error.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import (AppendParams, CompactParams, DecodeParams, GateParams, PikvError, check, lib)

PAGE_TOKENS = _lib.PAGE_TOKENS
HEAD_DIM = _lib.HEAD_DIM


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _req(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise PikvError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise PikvError(f"{name} must be {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _dtype_code(t: torch.Tensor, name: str) -> int:
    if t.dtype == torch.float32:
        return _lib.PIKV_F32
    if t.dtype == torch.bfloat16:
        return _lib.PIKV_BF16
    raise PikvError(f"{name}: dtype {t.dtype} not supported (float32 or bfloat16)")


_ws_cache: dict = {}


def _workspace(dev: torch.device, nbytes: int, tag: str) -> torch.Tensor:
    """Per-(device, stream, tag) scratch buffer, grown on demand and reused."""
    key = (dev.index, torch.cuda.current_stream().cuda_stream, tag)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        _ws_cache[key] = buf
    return buf


# ------------------------------------------------------------------ gate
@dataclass
class GateResult:
    probs: Optional[torch.Tensor]      # [T,E] fp32
    topk_idx: torch.Tensor             # [T,k] int32
    topk_w: torch.Tensor               # [T,k] fp32
    slot: torch.Tensor                 # [T,k] int32, -1 = dropped at capacity
    counts_k: torch.Tensor             # [k,E] int32
    prob_sum: torch.Tensor             # [E] fp32
    new_len: torch.Tensor              # [E] int32
    workspace: Optional[torch.Tensor] = None   # gate scratch owned by this result (route_append)

    @property
    def counts(self) -> torch.Tensor:
        return self.counts_k.sum(0)


def gate_fused(act: Optional[torch.Tensor] = None, w2: Optional[torch.Tensor] = None,
               b2: Optional[torch.Tensor] = None, *, logits: Optional[torch.Tensor] = None, top_k: int = 2,
               expert_mask: Optional[torch.Tensor] = None, mask_mode: int = _lib.MASK_SINGLE,
               correction: Optional[torch.Tensor] = None, temperature: float = 1.0, renorm_eps: float = 0.0,
               capacity: int = 0, slot_base: Optional[torch.Tensor] = None, want_probs: bool = True,
               out: Optional[GateResult] = None, phase: int = 0, _mlp=None) -> GateResult:
    """Fused gate tail; see pikv_gate_fused in include/pikv_b200.h.

    Give either (act [T,H], w2 [E,H], b2 [E]) or logits [T,E] fp32.  phase 1 (scoring kernel only) and
    phase 2 (slot finalisation only, same arguments, ordered after phase 1 by the caller) keep their state
    in out.workspace, which is allocated on first use and must not be shared between batches in flight.
    """
    if _mlp is not None:
        # gate_mlp_fused: act is the net's input x [T,K]; the kernel forms the hidden activations itself
        x, w1, b1 = _mlp
        x = _req(x, "x", torch.bfloat16)
        w1 = _req(w1, "w1", torch.bfloat16)
        w2 = _req(w2, "w2", torch.bfloat16)
        T, Kin = x.shape
        H, E = w1.shape[0], w2.shape[0]
        if w1.shape[1] != Kin or w2.shape[1] != H:
            raise PikvError(f"w1 is {tuple(w1.shape)}, w2 {tuple(w2.shape)}: expected [H,{Kin}] and [E,H]")
        dev, dt, act = x.device, _lib.PIKV_BF16, None
    elif logits is not None:
        logits = _req(logits, "logits", torch.float32)
        T, E = logits.shape
        H, dev, dt = 0, logits.device, _lib.PIKV_F32
    else:
        act = _req(act, "act")
        w2 = _req(w2, "w2", act.dtype)
        T, H = act.shape
        E = w2.shape[0]
        if w2.shape[1] != H:
            raise PikvError(f"w2 is {tuple(w2.shape)}, expected [E,{H}]")
        dev, dt = act.device, _dtype_code(act, "act")
    f32 = dict(dtype=torch.float32, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    if out is None:
        out = GateResult(
            probs=torch.empty(T, E, **f32) if want_probs else None,
            topk_idx=torch.empty(T, top_k, **i32), topk_w=torch.empty(T, top_k, **f32),
            slot=torch.empty(T, top_k, **i32), counts_k=torch.empty(top_k, E, **i32),
            prob_sum=torch.empty(E, **f32), new_len=torch.empty(E, **i32))
    nws = lib().pikv_gate_workspace_bytes(T, E, top_k)
    if phase != 0 or out.workspace is not None:
        if out.workspace is None or out.workspace.numel() < nws:
            if phase == 2:
                raise PikvError("gate phase 2 needs the result (and workspace) of the phase 1 call")
            out.workspace = torch.empty(nws, dtype=torch.uint8, device=dev)
        ws = out.workspace
    else:
        ws = _workspace(dev, nws, "gate")
    keep = []

    def f(t):
        if t is None:
            return None
        t = _req(t.to(torch.float32), "gate vector", torch.float32)
        keep.append(t)
        return _p(t)

    p = GateParams()
    p.act, p.w2, p.b2, p.logits_in = _p(act) if logits is None else None, _p(w2) if logits is None else None, \
        f(b2) if logits is None else None, _p(logits)
    if _mlp is not None:
        p.act = None
    p.dtype, p.T, p.H, p.E, p.top_k = dt, T, H, E, top_k
    p.expert_mask = f(expert_mask)
    p.mask_mode = mask_mode if expert_mask is not None else _lib.MASK_NONE
    p.correction = f(correction)
    p.temperature, p.renorm_eps, p.capacity = float(temperature), float(renorm_eps), int(capacity)
    if slot_base is not None:
        slot_base = _req(slot_base, "slot_base", torch.int32)
    p.slot_base = _p(slot_base)
    p.probs, p.topk_idx, p.topk_w, p.slot = _p(out.probs), _p(out.topk_idx), _p(out.topk_w), _p(out.slot)
    p.counts_k, p.prob_sum, p.new_len = _p(out.counts_k), _p(out.prob_sum), _p(out.new_len)
    p.workspace, p.workspace_bytes, p.phase = _p(ws), ws.numel(), int(phase)
    if _mlp is not None:
        b1f = f(b1)
        check(lib().pikv_gate_mlp_fused(C.byref(p), _p(x), Kin, _p(w1), b1f, _stream()), "pikv_gate_mlp_fused")
        return out
    check(lib().pikv_gate_fused(C.byref(p), _stream()), "pikv_gate_fused")
    return out


def gate_mlp_fused(x: torch.Tensor, w1: torch.Tensor, b1: Optional[torch.Tensor], w2: torch.Tensor,
                   b2: Optional[torch.Tensor], **kw) -> GateResult:
    """The whole gate net on tensor cores: relu(x @ w1.T + b1) @ w2.T + b2, then the tail of gate_fused (same
    keyword arguments and result); bf16 x [T,K], w1 [H,K], w2 [E,H].  See pikv_gate_mlp_fused."""
    return gate_fused(None, w2, b2, _mlp=(x, w1, b1), **kw)


def dispatch_scatter(g: GateResult, num_experts: int, capacity: int, position_mode: int = 0):
    """Dense [T,E,capacity] fp32 dispatch and combine tensors from a gate result."""
    T, k = g.topk_idx.shape
    dev = g.topk_idx.device
    d = torch.empty(T, num_experts, capacity, dtype=torch.float32, device=dev)
    c = torch.empty_like(d)
    check(lib().pikv_dispatch_scatter(_p(g.topk_idx), _p(g.topk_w), _p(g.slot), _p(g.counts_k), T, num_experts, k,
                                      capacity, position_mode, _p(d), _p(c), _stream()), "pikv_dispatch_scatter")
    return d, c


# ------------------------------------------------------------------ block-wide fake quantisation
def quant_block(x: torch.Tensor, group_size: int, qmin: int, qmax: int, symmetric: bool,
                params_in: Optional[torch.Tensor] = None, want_codes: bool = False, want_err: bool = True):
    """Returns (dq [N,H] fp32, q or None, params [G,2] fp32 (scale, zero point), sq_err [G] or None)."""
    x = _req(x, "x")
    N, H = x.shape
    G = (H + group_size - 1) // group_size
    dev = x.device
    dq = torch.empty(N, H, dtype=torch.float32, device=dev)
    q = torch.empty(N, H, dtype=torch.float32, device=dev) if want_codes else None
    params = torch.empty(G, 2, dtype=torch.float32, device=dev)
    err = torch.empty(G, dtype=torch.float32, device=dev) if want_err else None
    if params_in is not None:
        params_in = _req(params_in, "params_in", torch.float32)
    ws = _workspace(dev, lib().pikv_quant_block_workspace_bytes(N, H, group_size), "qb")
    check(lib().pikv_quant_block(_p(x), _dtype_code(x, "x"), N, H, group_size, qmin, qmax, int(bool(symmetric)),
                                 _p(params_in), _p(params), _p(dq), _p(q), _p(err), _p(ws), ws.numel(), _stream()),
          "pikv_quant_block")
    return dq, q, params, err


# ------------------------------------------------------------------ H2O
def h2o_accumulate(acc: torch.Tensor, ts: torch.Tensor, idx: Optional[torch.Tensor], w: torch.Tensor, now: float,
                   decay: float = 1.0, status: Optional[torch.Tensor] = None) -> None:
    """In place: acc[idx] += w ; ts[idx] = now (acc *= decay first when decay != 1)."""
    acc = _req(acc, "acc", torch.float32)
    ts = _req(ts, "ts", torch.float32)
    w = _req(w, "w", torch.float32)
    if idx is not None:
        idx = _req(idx, "idx", torch.int32)
    check(lib().pikv_h2o_accumulate(_p(acc), _p(ts), acc.numel(), _p(idx), _p(w), w.numel(), float(now), float(decay),
                                    _p(status), _stream()), "pikv_h2o_accumulate")


def h2o_select(acc: torch.Tensor, ts: torch.Tensor, num_heavy: int, num_recent: int,
               seg_len: Optional[torch.Tensor] = None, n: Optional[int] = None, want_idx: bool = True,
               as_bool: bool = True):
    """acc, ts: [segments, stride] fp32.  Returns (evict_mask bool [segments,stride], keep_idx int32
    [segments, min(stride, heavy+recent)] ascending (unused tail undefined), kept_count int32 [segments]).
    as_bool=False returns the kernel's uint8 mask as it is (no conversion kernel)."""
    acc = _req(acc, "acc", torch.float32)
    ts = _req(ts, "ts", torch.float32)
    if acc.dim() == 1:
        acc, ts = acc[None], ts[None]
    S, stride = acc.shape
    n = stride if n is None else n
    dev = acc.device
    mask = torch.empty(S, stride, dtype=torch.uint8, device=dev)
    ks = max(1, min(stride, num_heavy + num_recent))
    keep = torch.empty(S, ks, dtype=torch.int32, device=dev) if want_idx else None
    cnt = torch.empty(S, dtype=torch.int32, device=dev)
    if seg_len is not None:
        seg_len = _req(seg_len, "seg_len", torch.int32)
    check(lib().pikv_h2o_select(_p(acc), _p(ts), S, stride, _p(seg_len), n, num_heavy, num_recent, _p(mask), _p(keep),
                                ks, _p(cnt), _stream()), "pikv_h2o_select")
    return (mask.bool() if as_bool else mask), keep, cnt


def h2o_accumulate_attn(scores: torch.Tensor, lse: torch.Tensor, seq_len: Optional[torch.Tensor], n_kv: int,
                        acc: torch.Tensor) -> None:
    """In place: acc[b*n_kv+h, pos] += sum over the group's query heads of exp(scores - lse)."""
    scores = _req(scores, "scores", torch.float32)
    lse = _req(lse, "lse", torch.float32)
    acc = _req(acc, "acc", torch.float32)
    B, n_q, stride = scores.shape
    check(lib().pikv_h2o_accumulate_attn(_p(scores), stride, _p(lse), _p(seq_len), B, n_q, n_kv, _p(acc),
                                         acc.shape[-1], _stream()), "pikv_h2o_accumulate_attn")


# ------------------------------------------------------------------ low-rank projection
def lowrank_project(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, relu: bool = True,
                    residual: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """y[M,N] = act(x[M,K] @ w[N,K]^T + bias) (+ residual) on tcgen05 tensor cores; x, w bf16."""
    x = _req(x, "x", torch.bfloat16)
    w = _req(w, "w", torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise PikvError(f"w is {tuple(w.shape)}, expected [N,{K}]")
    if bias is not None:
        bias = _req(bias.to(torch.float32), "bias", torch.float32)
    if residual is not None:
        residual = _req(residual, "residual", torch.bfloat16)
    out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    code = _lib.PIKV_BF16 if out_dtype == torch.bfloat16 else _lib.PIKV_F32
    check(lib().pikv_lowrank_project(_p(x), _p(w), _p(bias), _p(residual), _p(out), code, M, N, K, int(bool(relu)),
                                     _stream()), "pikv_lowrank_project")
    return out


# ------------------------------------------------------------------ all-to-all records
def a2a_record_bytes(n_kv: int) -> int:
    return int(lib().pikv_a2a_record_bytes(n_kv))


def a2a_pack(k: torch.Tensor, v: torch.Tensor, n_kv: int, dst_seq: torch.Tensor, slot: torch.Tensor,
             n_records: int, send_pos: Optional[torch.Tensor] = None, seq_prefix: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Quantise (int8 symmetric, per token and head) and pack routed rows into records.  The record
    index of (token, j) is send_pos[t,j], or seq_prefix[dst_seq[t,j]] + slot[t,j] when send_pos is None."""
    k = _req(k, "k")
    v = _req(v, "v", k.dtype)
    T = k.shape[0]
    top_k = dst_seq.shape[1]
    nbytes = max(n_records, 1) * a2a_record_bytes(n_kv)
    buf = out if out is not None else torch.empty(nbytes, dtype=torch.uint8, device=k.device)
    if buf.numel() < nbytes:
        raise PikvError("a2a_pack: output buffer too small")
    if send_pos is not None:
        send_pos = _req(send_pos, "send_pos", torch.int32)
    if seq_prefix is not None:
        seq_prefix = _req(seq_prefix, "seq_prefix", torch.int32)
    check(lib().pikv_a2a_pack(_p(k), _p(v), _dtype_code(k, "k"), T, n_kv, top_k, _p(_req(dst_seq, "dst_seq", torch.int32)),
                              _p(_req(slot, "slot", torch.int32)), _p(seq_prefix), _p(send_pos), _p(buf), _stream()),
          "pikv_a2a_pack")
    return buf
