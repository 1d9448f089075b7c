"""The allocation-free decode-attention entry point against the regular one, through the C ABI.

Some callers cannot allocate device memory when they need attention (all of HBM already belongs to
their own page pool, or they sit inside a stream capture); pikv_decode_attn_q8_static keeps its
scratch for partial results in an array inside the library instead.  Two calls in a row must both reproduce the
regular entry point, which shows that the shared array carries nothing over between calls.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(lib_mod, cache, q, out, seq_len, splits, ws):
    p = lib_mod.DecodeParams()
    B, n_q, _ = q.shape
    p.q, p.out, p.B, p.n_q, p.n_kv = q.data_ptr(), out.data_ptr(), B, n_q, cache.n_kv
    p.seq_ids, p.seq_len, p.page_table = None, seq_len.data_ptr(), cache.page_table.data_ptr()
    p.num_seqs, p.max_pages, p.num_pages = cache.num_seqs, cache.max_pages, cache.num_pages
    p.k_codes, p.v_codes = cache.k_codes.data_ptr(), cache.v_codes.data_ptr()
    p.k_scale, p.v_scale = cache.k_scale.data_ptr(), cache.v_scale.data_ptr()
    p.splits, p.lse, p.scores, p.score_stride = splits, None, None, 0
    p.workspace, p.workspace_bytes = (ws.data_ptr(), ws.numel()) if ws is not None else (None, 0)
    p.status = cache.status.data_ptr()
    return p


def test_static_scratch_entry_point_matches_regular_one():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import pikv_b200
    from pikv_b200 import _lib
    lib = pikv_b200.lib()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    B, n_q, n_kv, ctx, splits = 3, 8, 2, 700, 4
    cache = pikv_b200.PagedKVCache(B, ctx, n_kv, device=dev)
    K = torch.randn(B * ctx, n_kv * 128, device=dev).bfloat16()
    V = torch.randn(B * ctx, n_kv * 128, device=dev).bfloat16()
    seq = torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(ctx)[:, None].contiguous()
    pos = torch.arange(ctx, dtype=torch.int32, device=dev).repeat(B)[:, None].contiguous()
    cache.append(K, V, seq, pos)
    seq_len = torch.tensor([700, 333, 16], dtype=torch.int32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(lib.pikv_decode_attn_workspace_bytes(B, n_q, n_kv, ctx, splits), dtype=torch.uint8, device=dev)
    for call in range(2):                                   # two calls in a row share the built-in array
        q = torch.randn(B, n_q, 128, device=dev).bfloat16()
        want, got = torch.empty_like(q), torch.empty_like(q)
        assert lib.pikv_decode_attn_q8(C.byref(_params(_lib, cache, q, want, seq_len, splits, ws)), stream) == 0
        rc = lib.pikv_decode_attn_q8_static(C.byref(_params(_lib, cache, q, got, seq_len, splits, None)), stream)
        assert rc == 0, lib.pikv_last_error()
        torch.cuda.synchronize()
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.abs(g - w).max() <= 1e-2 * np.abs(w).max()
        assert np.array_equal(g, w)                         # same kernels, same order: in fact identical
    cache.check_status()
    # a request beyond the built-in array is refused with a clear message, nothing is launched
    big = _params(_lib, cache, q, got, seq_len, 64, None)
    big.B, big.n_q = 4096, 64
    assert lib.pikv_decode_attn_q8_static(C.byref(big), stream) == -4
    assert b"built-in" in lib.pikv_last_error()
    assert lib.pikv_decode_attn_static_scratch_bytes() == 8 << 20
