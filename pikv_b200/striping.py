"""Where the rows of an (expert, stream) cache live on an expert-sharded box: host arithmetic.

The reference's expert parallelism gives each rank a contiguous block of experts
(core/distributed/distributed_pikv.py:91-96; `expert_placement` in
core/distributed/distributed_config.py:18).  With skewed routing that puts most of the KV bytes, and
most of every decode step, on the ranks that own the popular experts.  Here the cache of a pair
(expert e, stream s) is cut into stripes of `stripe` tokens and stripe c lives on rank

    owner(e, s, c) = (perm[e] + s + c) mod world

so that both the experts and the long caches of popular experts are spread evenly: a decode request
over a pair of length L touches ceil(L / stripe) stripes, i.e. every rank once L >= world * stripe.
On its owner a stripe is stored behind the owner's earlier stripes of the same pair:

    local_slot(pos) = (pos // stripe // world) * stripe + pos % stripe

The same formulas run inside the append kernel (pikv_kv_append_striped) and the decode planner
(the plan kernel of pikv_shard_decode_attn); this module is their host-side statement, used to size and lay out the page
pools and by the tests.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

PAGE_TOKENS = 16


@dataclass
class StripedLayout:
    num_experts: int
    num_streams: int
    world: int
    stripe: int                 # tokens per stripe: a power of two, a multiple of the page
    perm: np.ndarray            # [E] int32 rotation of every expert

    def __post_init__(self):
        if self.stripe < PAGE_TOKENS or self.stripe & (self.stripe - 1):
            raise ValueError("stripe must be a power of two and at least one page (16 tokens)")
        if not 1 <= self.world <= 8:
            raise ValueError("one box: 1 to 8 ranks")
        self.perm = np.asarray(self.perm, np.int32)
        if self.perm.shape != (self.num_experts,):
            raise ValueError("perm must have one entry per expert")

    # -- pairs ---------------------------------------------------------------------------------------
    @property
    def num_pairs(self) -> int:
        return self.num_experts * self.num_streams

    def pair(self, e, s):
        """Sequence id of (expert, stream): the same on every rank."""
        return np.asarray(e) * self.num_streams + np.asarray(s)

    def rot(self, e, s):
        return (self.perm[np.asarray(e)] + np.asarray(s)) % self.world

    def home(self, s):
        """Rank that gates and appends the tokens of stream s and issues its decode queries."""
        per = -(-self.num_streams // self.world)
        return np.asarray(s) // per

    # -- rows ----------------------------------------------------------------------------------------
    def owner(self, e, s, pos):
        return (self.rot(e, s) + np.asarray(pos) // self.stripe) % self.world

    def local_slot(self, pos):
        pos = np.asarray(pos)
        return (pos // self.stripe // self.world) * self.stripe + pos % self.stripe

    def local_len(self, e, s, length, rank):
        """Tokens of the first `length` positions of pair (e, s) that rank `rank` stores."""
        length = np.asarray(length, np.int64)
        full, tail = length // self.stripe, length % self.stripe
        first = (rank - self.rot(e, s)) % self.world            # this rank's first stripe of the pair
        n_full = np.where(full > first, (full - first + self.world - 1) // self.world, 0)
        mine_tail = (full % self.world) == first                 # the partial last stripe is stripe number `full`
        return n_full * self.stripe + np.where(mine_tail, tail, 0)

    # -- page pools ----------------------------------------------------------------------------------
    def local_capacity(self, cap_tokens):
        """Slots a rank must hold for a pair that may grow to cap_tokens: its share of the stripes, rounded
        up (ceil(stripes / world) stripes)."""
        stripes = -(-np.asarray(cap_tokens, np.int64) // self.stripe)
        return (-(-stripes // self.world)) * self.stripe

    def page_table(self, cap_by_expert):
        """Replicated page table [E * S, max_pages] (int32, -1 past a pair's allocation) and the number of
        pages per rank.  Every rank lays its pool out the same way, so an appender finds the page of a remote
        row in its own copy of the table."""
        cap_by_expert = np.asarray(cap_by_expert, np.int64)
        pages_e = self.local_capacity(cap_by_expert) // PAGE_TOKENS          # [E]
        per_pair = np.repeat(pages_e, self.num_streams)                       # pair = e * S + s
        start = np.concatenate([[0], np.cumsum(per_pair)])
        max_pages = int(pages_e.max())
        ar = np.arange(max_pages, dtype=np.int64)[None, :]
        table = np.where(ar < per_pair[:, None], start[:-1, None] + ar, -1).astype(np.int32)
        return table, int(start[-1])


def zipf_expert_logits(num_experts: int, exponent: float = 1.1) -> np.ndarray:
    """log of the Zipf(exponent) popularity of expert rank 1..E (the skew of the sharded configuration)."""
    p = 1.0 / np.arange(1, num_experts + 1, dtype=np.float64) ** exponent
    return np.log(p / p.sum()).astype(np.float32)
