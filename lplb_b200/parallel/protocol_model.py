"""Executable model of the in-kernel statistics exchange, for testing on a CPU.

The kernel protocol (``exchange_counts`` in ``csrc/planner_kernels.cuh``): in launch number
``n`` (the epoch) every rank stores, for each element, the word ``(n << 32) | count`` into
slot ``[n & 1][my_rank]`` of every rank's receive buffer, then polls its own buffer until
every word of parity ``n & 1`` carries tag ``n`` or a time budget runs out, summing the words
as they arrive (the sum replaces the rank's own vector in place).  A rank whose words did not
arrive in time is reported and replaced by the reader's own counts, which the reader takes
from its own slot of its receive buffer (it pushes to itself like to any peer).  The kernel
stores two adjacent words with one 16-byte store when the vector length is even; each half
carries its own tag, so the model's unit of delivery stays the single word.
With a node size the exchange runs in two levels, each with its own slots
``[n & 1][level][my_rank]``: first among the ranks of a node, then the node sums among the
ranks that hold the same position in every node (``two_level_step``).  Counts use 31 bits;
bit 31 of a vector's first word marks a node sum in which a late rank's share was replaced,
so that the other nodes report the timeout as well.

The model keeps the same state and lets a test decide, store by store, when (or whether)
each one is delivered: in order, late, twice, or never.  The only ordering assumed of the
fabric is the one the hardware gives: two stores from one source to one address are
delivered in program order.
"""

from __future__ import annotations

import random
from dataclasses import dataclass, field

__all__ = ["Fabric", "Rank", "run_lockstep", "two_level_step"]


@dataclass
class Store:
    src: int
    dst: int
    parity: int
    elem: int
    word: int
    level: int = 0


@dataclass
class Fabric:
    """In-flight stores, one FIFO per (src, dst, address)."""

    n_ranks: int
    n_elems: int
    queues: dict = field(default_factory=dict)
    dropped_sources: set = field(default_factory=set)

    def send(self, st: Store) -> None:
        if st.src in self.dropped_sources and st.dst != st.src:
            return
        self.queues.setdefault((st.src, st.dst, st.parity, st.elem, st.level), []).append(st)

    def pending(self) -> list:
        return [k for k, q in self.queues.items() if q]

    def deliver(self, key, ranks, duplicate: bool = False) -> None:
        st = self.queues[key][0] if duplicate else self.queues[key].pop(0)
        ranks[st.dst].recv[st.parity][st.level][st.src][st.elem] = st.word

    def deliver_all(self, ranks, rng: random.Random | None = None) -> None:
        keys = self.pending()
        while keys:
            key = rng.choice(keys) if rng else keys[0]
            self.deliver(key, ranks)
            keys = self.pending()


class Rank:
    def __init__(self, rank: int, n_ranks: int, n_elems: int):
        self.rank, self.n_ranks, self.n_elems = rank, n_ranks, n_elems
        self.epoch = 0
        # recv[parity][level][source rank][element]
        self.recv = [[[[0] * n_elems for _ in range(n_ranks)] for _ in range(2)] for _ in range(2)]
        self.mine: list[int] = [0] * n_elems

    def publish(
        self, counts: list[int], fabric: Fabric, level: int = 0, peers=None, bump: bool = True, degraded: bool = False
    ) -> int:
        """First half of a level: (bump the epoch and) push the words to ``peers`` (default: all).
        ``degraded`` sets bit 31 of the first word: "this vector contains a substituted share"."""
        if bump:
            self.epoch += 1
        self.mine = list(counts)
        for dst in range(self.n_ranks) if peers is None else peers:
            for e, c in enumerate(counts):
                low = (c & 0x7FFFFFFF) | (0x80000000 if degraded and e == 0 else 0)
                fabric.send(Store(self.rank, dst, self.epoch & 1, e, (self.epoch << 32) | low, level))
        return self.epoch

    def ready(self, level: int = 0) -> list[bool]:
        """Per source rank: do all words of the current parity carry the current epoch?"""
        buf = self.recv[self.epoch & 1][level]
        return [all((w >> 32) == self.epoch for w in buf[src]) for src in range(self.n_ranks)]

    def finish(self, level: int = 0, peers=None) -> tuple[list[int], int]:
        """Second half of a level: sum what arrived from ``peers``; returns ``(sums, missing bit mask)``."""
        peers = range(self.n_ranks) if peers is None else peers
        ok = self.ready(level)
        buf = self.recv[self.epoch & 1][level]
        miss = sum(1 << r for r in peers if not ok[r])
        # a vector that arrived but carries the degraded mark is used as it is and reported
        miss |= sum(1 << r for r in peers if ok[r] and buf[r][0] & 0x80000000)
        # the substitute for an absent rank is this rank's own vector as it sits in its own slot
        own = [
            (buf[self.rank][e] & 0x7FFFFFFF) if (buf[self.rank][e] >> 32) == self.epoch else self.mine[e]
            for e in range(self.n_elems)
        ]
        sums = [
            sum((buf[src][e] & 0x7FFFFFFF) if ok[src] else own[e] for src in peers)
            for e in range(self.n_elems)
        ]
        return sums, miss


def run_lockstep(n_ranks: int, n_elems: int, steps: int, seed: int = 0):
    """All ranks publish, the fabric delivers in random order, all ranks finish; repeated."""
    rng = random.Random(seed)
    ranks = [Rank(r, n_ranks, n_elems) for r in range(n_ranks)]
    fabric = Fabric(n_ranks, n_elems)
    history = []
    for _ in range(steps):
        counts = [[rng.randrange(0, 1 << 20) for _ in range(n_elems)] for _ in range(n_ranks)]
        for r in ranks:
            r.publish(counts[r.rank], fabric)
        fabric.deliver_all(ranks, rng)
        results = [r.finish() for r in ranks]
        history.append((counts, results))
    return history


def two_level_step(ranks, fabric: Fabric, counts, node_size: int, deliver=None):
    """One launch of the two-level schedule on every rank: node peers first, then the ranks
    with the same position in the other nodes.  ``deliver(level)`` moves stores between the
    publish and the finish of a level (default: everything, in order).  Returns per rank
    ``(sums, missing bit mask over both levels)``."""
    n = len(ranks)
    deliver = deliver or (lambda level: fabric.deliver_all(ranks))
    node_peers = [list(range(r // node_size * node_size, r // node_size * node_size + node_size)) for r in range(n)]
    cross_peers = [list(range(r % node_size, n, node_size)) for r in range(n)]
    for r in ranks:
        r.publish(counts[r.rank], fabric, level=0, peers=node_peers[r.rank])
    deliver(0)
    node_sums = [r.finish(0, node_peers[r.rank]) for r in ranks]
    for r in ranks:
        r.publish(
            node_sums[r.rank][0], fabric, level=1, peers=cross_peers[r.rank], bump=False,
            degraded=node_sums[r.rank][1] != 0,
        )
    deliver(1)
    out = []
    for r in ranks:
        sums, miss = r.finish(1, cross_peers[r.rank])
        out.append((sums, miss | node_sums[r.rank][1]))
    return out
