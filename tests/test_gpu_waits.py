"""Bounded waits that actually run out, made on the host side: one process plays rank 0 of a two-rank
exchange whose "peer" is a local buffer nobody writes, so the flag the kernel waits for is never raised.
With a 20 ms limit the kernel must come back with PIKV_ST_WAIT_TIMEOUT, drop the step's rows and mark
itself failed; nothing traps, hangs or faults, and the context stays usable."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
FAILED = 0x80000000


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _exchange(dev, E=8, top_k=2, capacity=100, limit_us=20000):
    from pikv_b200 import _lib
    W, ring = 2, _lib.XCHG_RING
    t = dict(
        counts_k=torch.arange(top_k * E, dtype=torch.int32, device=dev).view(top_k, E).contiguous(),
        gather=[torch.zeros(ring * W * E, dtype=torch.int32, device=dev) for _ in range(W)],
        flags=[torch.zeros(ring * W, dtype=torch.int32, device=dev) for _ in range(W)],
        seq=torch.zeros(1, dtype=torch.int32, device=dev), len_all=torch.zeros(E, dtype=torch.int32, device=dev),
        slot_base=torch.full((E,), -7, dtype=torch.int32, device=dev), status=torch.zeros(1, dtype=torch.int32, device=dev))
    p = _lib.ShardExchangeParams()
    p.counts_k, p.top_k, p.E, p.world, p.rank, p.capacity, p.start_empty = t["counts_k"].data_ptr(), top_k, E, W, 0, capacity, 0
    for r in range(W):
        p.peer_gather[r], p.peer_flags[r] = t["gather"][r].data_ptr(), t["flags"][r].data_ptr()
    p.seq, p.len_all, p.slot_base, p.status = t["seq"].data_ptr(), t["len_all"].data_ptr(), t["slot_base"].data_ptr(), t["status"].data_ptr()
    p.wait_limit_us = limit_us
    return p, t


def _call(p):
    import pikv_b200
    rc = pikv_b200.lib().pikv_shard_exchange_plan(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, pikv_b200.lib().pikv_last_error()
    torch.cuda.synchronize()


def test_count_exchange_wait_runs_out_and_failure_sticks(dev):
    from pikv_b200 import _lib
    p, t = _exchange(dev)
    E, W = 8, 2
    _call(p)                                                  # rank 1 never raises its flag
    assert int(t["status"].item()) & _lib.ST_WAIT_TIMEOUT
    assert (t["slot_base"] == 100).all()                      # every row of the step lands past the capacity: dropped
    assert (t["len_all"] == 0).all()                          # lengths untouched
    assert (int(t["seq"].item()) & 0xFFFFFFFF) == (1 | FAILED)
    # the rank's own counts went out before the wait (its peers may have used them)
    assert torch.equal(t["gather"][1].view(_lib.XCHG_RING, W, E)[1, 0], t["counts_k"].sum(0).to(torch.int32))
    # step 2: the peer's flag is there, but this rank is marked failed and stays so; its flag carries the mark
    t["status"].zero_()
    t["flags"][0][2 * W + 1] = 2
    _call(p)
    assert int(t["status"].item()) & _lib.ST_WAIT_TIMEOUT and (t["slot_base"] == 100).all()
    assert (int(t["flags"][1][2 * W + 0].item()) & 0xFFFFFFFF) == (2 | FAILED)
    # step 3 restarts the cache (start_empty) with the peer present: the marks clear and the plan is normal
    t["status"].zero_()
    t["flags"][0][3 * W + 1] = 3
    t["gather"][0].view(_lib.XCHG_RING, W, E)[3, 1] = 5       # rank 1 selected every expert five times
    p.start_empty = 1
    _call(p)
    assert int(t["status"].item()) == 0
    assert (int(t["seq"].item()) & 0xFFFFFFFF) == 3
    assert (t["slot_base"] == 0).all()                        # rank 0's rows come first
    assert torch.equal(t["len_all"], (t["counts_k"].sum(0) + 5).to(torch.int32))


def test_count_exchange_sees_a_failed_peer_at_once(dev):
    from pikv_b200 import _lib
    p, t = _exchange(dev, limit_us=5_000_000)                 # a long limit: the mark must end the wait, not the clock
    t["flags"][0][1 * 2 + 1] = torch.tensor(1 | FAILED, dtype=torch.int64).to(torch.int32)   # peer raised step 1, marked failed
    import time
    t0 = time.time()
    _call(p)
    assert time.time() - t0 < 2.0
    assert int(t["status"].item()) & _lib.ST_WAIT_TIMEOUT
    assert (t["slot_base"] == 100).all()
    assert (int(t["seq"].item()) & 0xFFFFFFFF) == (1 | FAILED)


def test_peer_barrier_wait_runs_out(dev):
    import pikv_b200
    from pikv_b200 import _lib
    flags = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
    seq, status = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    p = _lib.PeerBarrierParams()
    p.world, p.rank, p.seq, p.status, p.wait_limit_us = 2, 0, seq.data_ptr(), status.data_ptr(), 20000
    for r in range(2):
        p.peer_flags[r] = flags[r].data_ptr()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert pikv_b200.lib().pikv_peer_barrier(C.byref(p), st) == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _lib.ST_WAIT_TIMEOUT           # rank 1 never arrived
    assert int(flags[1][0].item()) == 1                        # rank 0's arrival was announced to rank 1
    status.zero_()
    flags[0][1] = 2                                            # rank 1 arrives at the second barrier
    assert pikv_b200.lib().pikv_peer_barrier(C.byref(p), st) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(seq.item()) == 2
    # the context is alive: an ordinary kernel still runs
    assert float(torch.ones(4, device=dev).sum().item()) == 4.0
