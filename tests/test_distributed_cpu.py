"""Host logic of the expert-sharded exchange on CPU ranks (gloo, world size 2): the exchange plan,
the record order and the owner-side slots must reproduce the single-process slot assignment."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _routing(T, E, k, seed):
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, E + 1) ** 1.1                    # Zipf-skewed expert popularity
    return np.stack([rng.choice(E, size=k, replace=False, p=p / p.sum()) for _ in range(T)]).astype(np.int64)


def _worker(rank, world, port, T, E, k, cap, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pikv_b200.distributed import plan_exchange, experts_per_rank
        from oracle import pikv_oracle as O
        idx_all = _routing(T, E, k, 0)
        per_rank = T // world
        idx = idx_all[rank * per_rank:(rank + 1) * per_rank]                  # contiguous split of the batch
        local_slot, counts_k = O.slot_assign_fast(idx, E, 1 << 30)              # what the gate returns with capacity 0
        counts = torch.from_numpy(counts_k.sum(0).astype(np.int32))
        gathered = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, counts)
        counts_all = torch.stack(gathered).numpy()
        per = experts_per_rank(E, world)
        plan = plan_exchange(counts_all, rank, np.zeros(per, np.int64), cap)
        # records = (global token, j, expert, local slot), placed at seq_prefix[expert] + local slot
        send = np.zeros((plan.n_send, 4), np.int64)
        for t in range(per_rank):
            for j in range(k):
                e = idx[t, j]
                send[plan.seq_prefix[e] + local_slot[t, j]] = (rank * per_rank + t, j, e, local_slot[t, j])
        recv = torch.zeros(plan.n_recv, 4, dtype=torch.int64)
        dist.all_to_all_single(recv, torch.from_numpy(send), output_split_sizes=plan.recv_splits.tolist(),
                               input_split_sizes=plan.send_splits.tolist())
        recv = recv.numpy()
        # owner-side slot of every received record
        final = np.full((T, k), -2, np.int64)
        for s in range(world):
            for i in range(plan.seg_start[s], plan.seg_start[s + 1]):
                tok, j, e, ls = recv[i]
                assert rank * per <= e < (rank + 1) * per                       # only experts this rank owns arrive
                slot = ls + plan.seg_base[s, e - rank * per]
                final[tok, j] = slot if slot < cap else -1
        np.save(os.path.join(tmp, f"final{rank}.npy"), final)
        np.save(os.path.join(tmp, f"len{rank}.npy"), plan.new_len)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T,E,k,cap", [(256, 8, 2, 1 << 20), (300, 4, 2, 90)])
def test_sharded_exchange_reproduces_single_process_slots(tmp_path, T, E, k, cap):
    from oracle import pikv_oracle as O
    world = 2
    T = T - T % world
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, T, E, k, cap, str(tmp_path)), nprocs=world, join=True)
    idx_all = _routing(T, E, k, 0)
    want, counts_k = O.slot_assign_fast(idx_all, E, cap)
    got = np.full((T, k), -2, np.int64)
    per = E // world
    for r in range(world):
        f = np.load(tmp_path / f"final{r}.npy")
        own = (idx_all >= r * per) & (idx_all < (r + 1) * per)
        got[own] = f[own]
        np.testing.assert_array_equal(np.load(tmp_path / f"len{r}.npy"),
                                      np.minimum(counts_k.sum(0)[r * per:(r + 1) * per], cap))
    np.testing.assert_array_equal(got, want)


def test_plan_exchange_shapes():
    from pikv_b200.distributed import plan_exchange
    counts = np.array([[3, 1, 0, 2], [1, 1, 4, 0]])
    p = plan_exchange(counts, 1, np.array([5, 0]), 8)
    np.testing.assert_array_equal(p.send_splits, [2, 4])          # rank 1 sends 1+1 to rank 0, 4+0 to itself
    np.testing.assert_array_equal(p.recv_splits, [2, 4])          # experts 2,3: from rank 0: 0+2, from rank 1: 4+0
    np.testing.assert_array_equal(p.seq_prefix, [0, 1, 2, 6])
    np.testing.assert_array_equal(p.seg_start, [0, 2, 6])
    np.testing.assert_array_equal(p.seg_base, [[5, 0], [5, 2]])
    np.testing.assert_array_equal(p.new_len, [8, 2])              # 5 + 4 = 9 truncated at capacity 8


def _peer_worker(rank, world, port, T, E, k, cap, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pikv_b200.distributed import experts_per_rank
        from oracle import pikv_oracle as O
        per = experts_per_rank(E, world)
        per_rank = T // world
        lengths = np.zeros(E, np.int64)
        final_steps, runs_steps = [], []
        for step in range(2):                                               # two steps: lengths carry over
            idx = _routing(T, E, k, step)[rank * per_rank:(rank + 1) * per_rank]
            local_slot, counts_k = O.slot_assign_fast(idx, E, 1 << 30)
            counts = counts_k.sum(0)
            gathered = [torch.zeros(E, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(counts.astype(np.int64)))
            base, lengths_new = O.shard_slot_base(torch.stack(gathered).numpy(), rank, lengths, cap)
            final = base[idx] + local_slot
            final[final >= cap] = -1
            final_steps.append(final)
            runs_steps.append(np.array(O.scale_push_runs(base, counts, cap, lambda e: e // per, rank), np.int64).reshape(-1, 4))
            lengths = lengths_new
        np.save(os.path.join(tmp, f"peer_final{rank}.npy"), np.stack(final_steps))
        np.save(os.path.join(tmp, f"peer_len{rank}.npy"), lengths)
        for i, r in enumerate(runs_steps):
            np.save(os.path.join(tmp, f"peer_runs{rank}_{i}.npy"), r)
    finally:
        dist.destroy_process_group()


def test_peer_exchange_slots_equal_single_process(tmp_path):
    """The slot arithmetic of the peer-store variant (count exchange, slot base per rank, scale runs) on two
    gloo ranks against the single-process slot assignment over the concatenated batch."""
    from oracle import pikv_oracle as O
    world, T, E, k, cap = 2, 600, 8, 2, 260
    mp.spawn(_peer_worker, args=(world, 29800 + os.getpid() % 1000, T, E, k, cap, str(tmp_path)), nprocs=world, join=True)
    lengths = np.zeros(E, np.int64)
    per, per_rank = E // world, T // world
    for step in range(2):
        idx = _routing(T, E, k, step)
        # single process: running count per expert over (token, k) order, on top of the lengths so far
        slot = np.full((T, k), -1, np.int64)
        run = lengths.copy()
        for t in range(T):
            for j in range(k):
                e = idx[t, j]
                slot[t, j] = run[e] if run[e] < cap else -1
                run[e] += 1
        got = np.concatenate([np.load(tmp_path / f"peer_final{r}.npy")[step] for r in range(world)])
        np.testing.assert_array_equal(got, slot)
        # scale runs: every remote (expert, slot) a rank wrote appears in exactly one of its runs, nothing else does
        for r in range(world):
            mine = set()
            part = slice(r * per_rank, (r + 1) * per_rank)
            for e, s_ in zip(idx[part].reshape(-1), slot[part].reshape(-1)):
                if s_ >= 0 and e // per != r:
                    mine.add((int(e), int(s_)))
            covered = set()
            for e, p, lo, hi in np.load(tmp_path / f"peer_runs{r}_{step}.npy"):
                for row in range(lo, hi):
                    assert (int(e), int(p * 16 + row)) not in covered
                    covered.add((int(e), int(p * 16 + row)))
            assert covered == mine
        lengths = np.minimum(run, cap)
    for r in range(world):
        np.testing.assert_array_equal(np.load(tmp_path / f"peer_len{r}.npy"), lengths)


def _failing_worker(rank, world, port, tmp):
    """Rank 1 raises before the count exchange; rank 0 must get an error out of its collective (a short
    process-group timeout), not wait for ever."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    outcome = "no error"
    try:
        if rank == 1:
            raise RuntimeError("injected failure on rank 1 (host side)")
        counts = torch.ones(8, dtype=torch.int32)
        gathered = [torch.zeros(8, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, counts)                    # the peer never joins
    except RuntimeError as e:
        outcome = "injected" if "injected" in str(e) else "collective error"
    except Exception:
        outcome = "collective error"
    with open(os.path.join(tmp, f"outcome{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)            # skip destroy_process_group: the peer is gone, and a clean shutdown would wait for it


def test_rank_failure_surfaces_as_an_error_on_the_other_rank(tmp_path):
    world = 2
    ctx = mp.get_context("spawn")
    port = 29800 + os.getpid() % 1000
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0, "a rank hung or crashed"
    assert (tmp_path / "outcome1.txt").read_text() == "injected"
    assert (tmp_path / "outcome0.txt").read_text() == "collective error"
