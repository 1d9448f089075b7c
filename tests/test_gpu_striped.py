"""The striped expert-sharded cache with all ranks emulated on one GPU (their buffers are local tensors and
each phase runs for every rank before the next one starts, so no kernel waits for one that has not run):
the ranks' rows together are the rows of ONE cache over all (expert, stream) pairs, bit for bit, and a decode
step over the ranks equals the oracle's routed combine and the single-cache result."""
import numpy as np
import pytest
import torch

from oracle import pikv_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _build(dev, world, stripe, E=6, S=8, n_kv=2, n_q=8, k=2, rounds=2, seed=0):
    import pikv_b200
    from pikv_b200 import ops
    from pikv_b200.striping import StripedLayout, zipf_expert_logits
    from pikv_b200.striped_cache import emulate_ranks
    rng = np.random.default_rng(seed)
    lay = StripedLayout(E, S, world, stripe, rng.permutation(E))
    cap = np.array([260, 200, 150, 90, 64, 33][:E])                # tight for the popular experts: rows get dropped
    ranks = emulate_ranks(lay, n_kv, n_q, k, cap, dev)
    single = pikv_b200.PagedKVCache(E * S, int(cap.max()), n_kv, device=dev)
    base = torch.from_numpy(zipf_expert_logits(E)).to(dev)
    g = torch.Generator(device=dev).manual_seed(seed)
    lens = torch.zeros(S, E, dtype=torch.int32, device=dev)
    capt = torch.from_numpy(cap.astype(np.int32)).to(dev)
    for _ in range(rounds):
        for s in range(S):
            T = int(rng.integers(40, 200))
            logits = (base[None] + torch.randn(T, E, generator=g, device=dev)).contiguous()
            K = torch.randn(T, n_kv * 128, generator=g, device=dev).bfloat16()
            V = torch.randn(T, n_kv * 128, generator=g, device=dev).bfloat16()
            home = ranks[int(lay.home(s))]
            res = home.route_append(s, K, V, logits=logits)
            # the same rows into one cache over all pairs: sequence = pair id, slot = position, cut at the capacity
            slot = torch.where(res.slot < capt[res.topk_idx.long()], res.slot, torch.full_like(res.slot, -1))
            single.append(K, V, (res.topk_idx * S + s).to(torch.int32), slot)
            lens[s] = torch.minimum(res.new_len, capt)
    torch.cuda.synchronize()
    for r in ranks:
        r.check_status()
    single.check_status()
    return lay, ranks, single, lens.cpu().numpy(), cap


@pytest.mark.parametrize("world,stripe", [(1, 64), (2, 32), (4, 16), (8, 32)])
def test_striped_append_rows_equal_single_cache(dev, world, stripe):
    lay, ranks, single, lens, cap = _build(dev, world, stripe)
    E, S = lay.num_experts, lay.num_streams
    assert lens.max() == cap.max() and (lens <= cap[None]).all()      # the hot experts hit their capacity
    for r, rk in enumerate(ranks):
        np.testing.assert_array_equal(rk.pair_len.cpu().numpy(), lens[r * rk.streams_per_rank:(r + 1) * rk.streams_per_rank])
    total = 0
    for e in range(E):
        for s in range(S):
            n = int(lens[s, e])
            if n == 0:
                continue
            pos = np.arange(n)
            own, loc = lay.owner(e, s, pos), lay.local_slot(pos)
            pair = torch.full((n,), e * S + s, dtype=torch.int32, device=dev)
            for which in ("k", "v"):
                want_dq, want = single.gather(pair, torch.from_numpy(pos.astype(np.int32)).to(dev), which, codes=True)
                for r, rk in enumerate(ranks):
                    m = own == r
                    if not m.any():
                        continue
                    mi = torch.from_numpy(np.nonzero(m)[0]).to(dev)
                    dq, got = rk.gather(pair[mi], torch.from_numpy(loc[m].astype(np.int32)).to(dev), which, codes=True)
                    assert torch.equal(got, want[mi]), (e, s, r, which)
                    assert torch.equal(dq, want_dq[mi])               # the scales arrived too
            total += n
    assert total == lens.sum()


@pytest.mark.parametrize("world,stripe,mode", [(1, 64, 0), (2, 32, 0), (4, 16, 1), (8, 32, 0), (4, 32, 0)])
def test_striped_decode_step_matches_oracle_and_single_cache(dev, world, stripe, mode):
    from pikv_b200 import ops
    from pikv_b200.striping import zipf_expert_logits
    lay, ranks, single, lens, cap = _build(dev, world, stripe, seed=3)
    E, S, k = lay.num_experts, lay.num_streams, 2
    n_q, n_kv = ranks[0].n_q, ranks[0].n_kv
    g = torch.Generator(device=dev).manual_seed(9)
    q = torch.randn(S, n_q, 128, generator=g, device=dev).bfloat16()
    logits = (torch.from_numpy(zipf_expert_logits(E)).to(dev)[None] + torch.randn(S, E, generator=g, device=dev)).contiguous()
    route = ops.gate_fused(logits=logits, top_k=k, capacity=0)
    spr = ranks[0].streams_per_rank
    for phase in ("post", "attend", "combine"):                       # every rank finishes a phase before the next starts
        outs = []
        for r, rk in enumerate(ranks):
            sl = slice(r * spr, (r + 1) * spr)
            if phase == "post":
                rk.decode_post(q[sl].contiguous(), route.topk_idx[sl].contiguous(), route.topk_w[sl].contiguous())
            elif phase == "attend":
                rk.decode_attend()
            else:
                outs.append(rk.decode_combine(mode=mode))
    torch.cuda.synchronize()
    for rk in ranks:
        rk.check_status()
    got = torch.cat(outs).float().cpu().numpy()
    # the oracle on the dequantised single cache
    ctx = int(cap.max())
    kd = np.zeros((E, S, n_kv, ctx, 128), np.float32)
    vd = np.zeros_like(kd)
    for e in range(E):
        for s in range(S):
            n = int(lens[s, e])
            if n:
                pair = torch.full((n,), e * S + s, dtype=torch.int32, device=dev)
                pos = torch.arange(n, dtype=torch.int32, device=dev)
                kd[e, s, :, :n] = single.gather(pair, pos, "k").cpu().numpy().reshape(n, n_kv, 128).transpose(1, 0, 2)
                vd[e, s, :, :n] = single.gather(pair, pos, "v").cpu().numpy().reshape(n, n_kv, 128).transpose(1, 0, 2)
    idx, w = route.topk_idx.cpu().numpy(), route.topk_w.cpu().numpy()
    want = O.routed_decode_combine(q.float().cpu().numpy(), kd, vd, lens.T, idx, w, lse_merge=bool(mode))
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    if mode == 0:
        # and the single-cache path: one decode call over the S x k (stream, choice) requests, weighted sum
        seq_ids = (route.topk_idx * S + torch.arange(S, device=dev, dtype=torch.int32)[:, None]).reshape(-1).contiguous()
        qq = q[:, None].expand(S, k, n_q, 128).reshape(S * k, n_q, 128).contiguous()
        o = single.decode_attention(qq, seq_ids=seq_ids, seq_len=torch.from_numpy(lens).to(dev)[
            torch.arange(S, device=dev)[:, None], route.topk_idx.long()].reshape(-1).to(torch.int32).contiguous())
        ref = (o.float().view(S, k, n_q, 128) * route.topk_w[:, :, None, None]).sum(1).cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()
