"""Host arithmetic of the striped (expert, stream) placement against brute force and the oracle's statement."""
import numpy as np
import pytest

from oracle import pikv_oracle as O
from pikv_b200.striping import StripedLayout, zipf_expert_logits


@pytest.mark.parametrize("world,stripe", [(1, 64), (2, 32), (4, 16), (8, 128)])
def test_every_row_has_one_owner_and_local_slots_are_dense(world, stripe):
    rng = np.random.default_rng(world)
    E, S = 6, 5
    lay = StripedLayout(E, S, world, stripe, rng.permutation(E))
    for e in range(E):
        for s in range(S):
            L = int(rng.integers(0, 5 * world * stripe))
            pos = np.arange(L)
            own, loc = lay.owner(e, s, pos), lay.local_slot(pos)
            o2, l2 = O.striped_owner(lay.perm, e, s, pos, stripe, world)
            np.testing.assert_array_equal(own, o2)
            np.testing.assert_array_equal(loc, l2)
            total = 0
            for r in range(world):
                mine = np.sort(loc[own == r])
                n = int(lay.local_len(e, s, L, r))
                assert n == len(mine)
                np.testing.assert_array_equal(mine, np.arange(n))        # dense: slots 0 .. n-1, in position order
                assert n <= lay.local_capacity(max(L, 1))
                total += n
            assert total == L


def test_page_table_is_a_partition_of_the_pool():
    lay = StripedLayout(4, 3, 2, 32, np.arange(4))
    cap = np.array([100, 64, 1, 33])
    table, pages = lay.page_table(cap)
    assert table.shape[0] == 12
    used = table[table >= 0]
    np.testing.assert_array_equal(np.sort(used), np.arange(pages))
    per_pair = (table >= 0).sum(1)
    np.testing.assert_array_equal(per_pair, np.repeat(lay.local_capacity(cap) // 16, 3))


def test_striping_balances_a_zipf_decode_step():
    """256 streams, 64 experts, Zipf(1.1) popularity: the hottest rank's share of a decode step's KV bytes
    stays within a few percent of the mean at 8 ranks (contiguous expert blocks: several times the mean)."""
    rng = np.random.default_rng(0)
    E, S, W, ctx = 64, 256, 8, 16384
    base = zipf_expert_logits(E)
    lay = StripedLayout(E, S, W, 1024, rng.permutation(E))
    lengths = np.zeros((E, S), np.int64)
    for s in range(S):
        top2 = np.argsort(-(base[None] + rng.standard_normal((ctx, E)).astype(np.float32)), axis=1)[:, :2]
        lengths[:, s] = np.bincount(top2.ravel(), minlength=E)
    qtop = np.argsort(-(base[None] + rng.standard_normal((S, E))), axis=1)[:, :2]
    load = np.zeros(W)
    block = np.zeros(W)
    for s in range(S):
        for e in qtop[s]:
            for r in range(W):
                load[r] += lay.local_len(e, s, lengths[e, s], r)
            block[e // (E // W)] += lengths[e, s]
    assert load.sum() == block.sum()
    assert load.max() / load.mean() < 1.06
    assert block.max() / block.mean() > 2.0
