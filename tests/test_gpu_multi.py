"""Two-GPU check of the expert-sharded exchange: the union of the two ranks' caches equals the cache a
single GPU builds from the concatenated batch.  Skipped with fewer than two GPUs."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmp, mode="a2a"):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from pikv_b200.distributed import ExpertShardedKVCache, PeerShardedKVCache
        T, H, E, k, n_kv = 2048, 512, 8, 2, 2
        cap = 900
        g = torch.Generator().manual_seed(7)
        act = torch.randn(T, H, generator=g).bfloat16()
        K = torch.randn(T, n_kv * 128, generator=g).bfloat16()
        V = torch.randn(T, n_kv * 128, generator=g).bfloat16()
        w2 = (torch.randn(E, H, generator=g) / 20).bfloat16().to(dev)
        per = T // world
        sl = slice(rank * per, (rank + 1) * per)
        peer = mode.startswith("peer")
        shard = (PeerShardedKVCache if peer else ExpertShardedKVCache)(E, cap, n_kv, dev)
        extra = {"split": True} if mode == "peer_split" else {}     # local and remote rows as two launches
        shard.route_append(act[sl].to(dev), w2, None, K[sl].to(dev), V[sl].to(dev), top_k=k, **extra)
        if peer:                # a second step on top of the first: lengths and bases carry over
            shard.route_append(act[sl].to(dev), w2, None, K[sl].to(dev), V[sl].to(dev), top_k=k, **extra)
        torch.cuda.synchronize()
        shard.cache.check_status()
        torch.save({n: getattr(shard.cache, n).cpu() for n in ("k_codes", "v_codes", "k_scale", "v_scale", "length")},
                   os.path.join(tmp, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["a2a", "peer", "peer_split"])
def test_two_gpu_cache_equals_single_gpu_cache(tmp_path, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import pikv_b200
    from pikv_b200 import ops
    world = 2
    mp.spawn(_worker, args=(world, 29600 + os.getpid() % 1000, str(tmp_path), mode), nprocs=world, join=True)
    dev = torch.device("cuda:0")
    T, H, E, k, n_kv, cap = 2048, 512, 8, 2, 2, 900
    g = torch.Generator().manual_seed(7)
    act = torch.randn(T, H, generator=g).bfloat16().to(dev)
    K = torch.randn(T, n_kv * 128, generator=g).bfloat16().to(dev)
    V = torch.randn(T, n_kv * 128, generator=g).bfloat16().to(dev)
    w2 = (torch.randn(E, H, generator=g) / 20).bfloat16().to(dev)
    res = ops.gate_fused(act, w2, None, top_k=k, capacity=cap)
    single = pikv_b200.PagedKVCache(E, cap, n_kv, device=dev)
    single.append(K, V, res.topk_idx, res.slot)
    if mode.startswith("peer"):  # the same batch appended twice, as the workers did
        res = ops.gate_fused(act, w2, None, top_k=k, capacity=cap, slot_base=res.new_len)
        single.append(K, V, res.topk_idx, res.slot)
    per = E // world
    pages = single.max_pages
    for r in range(world):
        got = torch.load(tmp_path / f"rank{r}.pt")
        for n in ("k_codes", "v_codes", "k_scale", "v_scale"):
            want = getattr(single, n)[r * per * pages:(r + 1) * per * pages].cpu()
            assert torch.equal(got[n], want), (r, n)
        assert torch.equal(got["length"], res.new_len[r * per:(r + 1) * per].cpu())


def _striped_worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from pikv_b200 import ops
        from pikv_b200.striping import StripedLayout
        from pikv_b200.striped_cache import StripedShardedKVCache
        E, S, n_kv, n_q, k, stripe = 6, 8, 2, 8, 2, 32
        lay = StripedLayout(E, S, world, stripe, np.random.default_rng(0).permutation(E))
        cap = np.array([260, 200, 150, 90, 64, 33])
        cache = StripedShardedKVCache.create(lay, n_kv, n_q, k, cap, dev, wait_limit_us=2_000_000)
        base = torch.log(torch.tensor([0.4, 0.25, 0.15, 0.1, 0.06, 0.04])).to(dev)
        for s in range(S):
            if int(lay.home(s)) != rank:
                continue
            g = torch.Generator(device=dev).manual_seed(100 + s)
            T = 150 + 10 * s
            logits = (base[None] + torch.randn(T, E, generator=g, device=dev)).contiguous()
            K = torch.randn(T, n_kv * 128, generator=g, device=dev).bfloat16()
            V = torch.randn(T, n_kv * 128, generator=g, device=dev).bfloat16()
            cache.route_append(s, K, V, logits=logits)
        cache.barrier()                                        # every rank's rows are in place
        g = torch.Generator(device=dev).manual_seed(7)
        q = torch.randn(S, n_q, 128, generator=g, device=dev).bfloat16()
        dl = (base[None] + torch.randn(S, E, generator=g, device=dev)).contiguous()
        route = ops.gate_fused(logits=dl, top_k=k, capacity=0)
        spr = cache.streams_per_rank
        sl = slice(rank * spr, (rank + 1) * spr)
        outs = []
        for step in range(2):                                  # two steps in a row: the flags carry step numbers
            outs.append(cache.decode_step(q[sl].contiguous(), route.topk_idx[sl].contiguous(), route.topk_w[sl].contiguous()).clone())
        torch.cuda.synchronize()
        cache.check_status()
        torch.save({"out0": outs[0].cpu(), "out1": outs[1].cpu(), "pair_len": cache.pair_len.cpu()}, os.path.join(tmp, f"striped{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_gpu_striped_cache_decode_equals_one_gpu(tmp_path):
    """The striped (expert, stream) cache on two GPUs (rows and decode partials crossing NVLink through peer
    stores and flags) against the same streams in a one-GPU cache: pair lengths equal, decode output within 1e-2."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from pikv_b200 import ops
    from pikv_b200.striping import StripedLayout
    from pikv_b200.striped_cache import emulate_ranks
    world = 2
    mp.spawn(_striped_worker, args=(world, 29700 + os.getpid() % 1000, str(tmp_path)), nprocs=world, join=True)
    dev = torch.device("cuda:0")
    E, S, n_kv, n_q, k, stripe = 6, 8, 2, 8, 2, 32
    perm = np.random.default_rng(0).permutation(E)
    cap = np.array([260, 200, 150, 90, 64, 33])
    one = emulate_ranks(StripedLayout(E, S, 1, stripe, perm), n_kv, n_q, k, cap, dev)[0]
    base = torch.log(torch.tensor([0.4, 0.25, 0.15, 0.1, 0.06, 0.04])).to(dev)
    for s in range(S):
        g = torch.Generator(device=dev).manual_seed(100 + s)
        T = 150 + 10 * s
        logits = (base[None] + torch.randn(T, E, generator=g, device=dev)).contiguous()
        K = torch.randn(T, n_kv * 128, generator=g, device=dev).bfloat16()
        V = torch.randn(T, n_kv * 128, generator=g, device=dev).bfloat16()
        one.route_append(s, K, V, logits=logits)
    g = torch.Generator(device=dev).manual_seed(7)
    q = torch.randn(S, n_q, 128, generator=g, device=dev).bfloat16()
    dl = (base[None] + torch.randn(S, E, generator=g, device=dev)).contiguous()
    route = ops.gate_fused(logits=dl, top_k=k, capacity=0)
    want = one.decode_step(q, route.topk_idx, route.topk_w).float().cpu()
    got = [torch.load(tmp_path / f"striped{r}.pt") for r in range(world)]
    assert torch.equal(torch.cat([x["pair_len"] for x in got]), one.pair_len.cpu())
    for key in ("out0", "out1"):
        full = torch.cat([x[key] for x in got]).float()
        assert float((full - want).abs().max()) <= 1e-2 * float(want.abs().max()), key
