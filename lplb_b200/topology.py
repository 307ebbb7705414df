"""Redundancy topologies (`r2o` matrices) and their validation.

An `r2o` matrix has shape ``[G, D]``: rank ``i``'s ``d``-th redundant slot holds a
copy of the ``d``-th replicated expert bundle of rank ``r2o[i, d]``.  Every column
must be a permutation of ``0..G-1`` so that each bundle has exactly one replica and
the inverse map ``o2r`` (origin -> replica holder) exists.

The reference ships these shapes only as test constants
(reference ``tests/utils.py:97-119``); here they are library functions, generated
from the graph they describe rather than written out as literals.
"""

from __future__ import annotations

from typing import Sequence

import torch

__all__ = [
    "ring",
    "circulant",
    "cube",
    "hypercube",
    "torus",
    "validate_r2o",
    "invert_r2o",
    "edge_list",
    "TOPOLOGIES",
    "by_name",
]


def _as_tensor(columns: Sequence[Sequence[int]]) -> torch.Tensor:
    """columns[d][i] = source rank of rank i's d-th redundant slot -> ``[G, D]``."""
    return torch.tensor(columns, dtype=torch.int32).T.contiguous()


def ring(n: int = 8) -> torch.Tensor:
    """One redundant slot per rank, copied from the next rank around a ring.

    Same graph as the reference's ``RING_8P`` for ``n == 8``
    (reference ``tests/utils.py:103-107``).
    """
    if n < 2:
        raise ValueError("a ring needs at least 2 ranks")
    return _as_tensor([[(i + 1) % n for i in range(n)]])


def circulant(n: int, shifts: Sequence[int] = (1,)) -> torch.Tensor:
    """``len(shifts)`` redundant slots per rank: slot ``d`` copies from the rank ``shifts[d]``
    places further around a ring of ``n`` ranks.  ``circulant(n, (1,))`` is ``ring(n)``; more
    shifts give denser graphs for any number of ranks and replicas (the reference has no
    generator for those; its shapes are the literals of reference ``tests/utils.py:97-119``).
    """
    if n < 2 or not shifts:
        raise ValueError("a circulant topology needs at least 2 ranks and 1 shift")
    if any(s % n == 0 for s in shifts):
        raise ValueError("a shift that is a multiple of the rank count is a self edge")
    return _as_tensor([[(i + s) % n for i in range(n)] for s in shifts])


def _quad_shift(n: int) -> list[int]:
    """Within each block of four ranks, take from the previous rank (cyclic)."""
    return [(i // 4) * 4 + (i + 3) % 4 for i in range(n)]


def cube() -> torch.Tensor:
    """8 ranks, 2 redundant slots per rank: two 4-cycles plus diagonal links.

    Slot 0 follows a 4-cycle inside each half.  Slot 1 crosses halves: the lower half
    takes from the diagonally opposite position of the upper half, the upper half
    takes from the same position of the lower half, which closes two more 4-cycles
    (0 6 2 4) and (1 7 3 5).  Same graph as the reference's ``CUBE_8P2E``
    (reference ``tests/utils.py:97-102``).
    """
    col1 = [4 + (i ^ 2) if i < 4 else i - 4 for i in range(8)]
    return _as_tensor([_quad_shift(8), col1])


def hypercube() -> torch.Tensor:
    """16 ranks, 2 redundant slots per rank, no diagonal links.

    Slot 0 follows a 4-cycle inside each block of four; slot 1 takes from the same
    position in the previous block of four (cyclic).  Same graph as the reference's
    ``HYPERCUBE_16P2E`` (reference ``tests/utils.py:108-113``).
    """
    col1 = [(i + 12) % 16 for i in range(16)]
    return _as_tensor([_quad_shift(16), col1])


def torus(m: int, n: int) -> torch.Tensor:
    """``m`` nodes of ``n`` ranks: slot 0 from the same position on the next node,
    slot 1 from the next rank on the same node.

    Same graph as the reference's ``torus_2d(m, n)`` (reference ``tests/utils.py:116-119``).
    """
    if m < 1 or n < 1 or m * n < 2:
        raise ValueError("torus needs at least 2 ranks")
    rows = []
    for node in range(m):
        for pos in range(n):
            rows.append([((node + 1) % m) * n + pos, node * n + (pos + 1) % n])
    return torch.tensor(rows, dtype=torch.int32)


def validate_r2o(r2o: torch.Tensor, *, allow_self_edges: bool = False) -> None:
    """Raise ``ValueError`` unless every column of ``r2o`` is a permutation of ranks.

    The reference never checks this; it silently computes ``argsort`` of a
    non-permutation (reference ``lplb/planner.py:66-68``).
    """
    if r2o.dim() != 2:
        raise ValueError(f"r2o must be [group_size, num_redundants], got {tuple(r2o.shape)}")
    g, d = r2o.shape
    if g < 1 or d < 1:
        raise ValueError("r2o must be non-empty")
    cpu = r2o.detach().to("cpu", torch.int64)
    want = torch.arange(g)
    for col in range(d):
        if not torch.equal(cpu[:, col].sort().values, want):
            raise ValueError(f"column {col} of r2o is not a permutation of 0..{g - 1}")
        if not allow_self_edges and bool((cpu[:, col] == want).any()):
            raise ValueError(f"column {col} of r2o has a rank replicating its own expert")


def invert_r2o(r2o: torch.Tensor) -> torch.Tensor:
    """``o2r[j, d]`` = the rank that holds the replica of rank ``j``'s ``d``-th bundle."""
    g, d = r2o.shape
    src = r2o.to(torch.int64)
    o2r = torch.empty_like(src)
    o2r.scatter_(0, src, torch.arange(g, device=r2o.device).unsqueeze(1).expand(g, d))
    return o2r.to(torch.int32).contiguous()


def edge_list(r2o: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Return ``(origin, holder)`` rank of every LP variable ``k = j*D + d``."""
    g, d = r2o.shape
    origin = torch.arange(g, dtype=torch.int64).unsqueeze(1).expand(g, d).reshape(-1)
    holder = invert_r2o(r2o.cpu()).to(torch.int64).reshape(-1)
    return origin, holder


TOPOLOGIES = {
    "ring8": lambda: ring(8),
    "cube": cube,
    "hypercube": hypercube,
    "torus8x4": lambda: torus(8, 4),
    "torus2x4": lambda: torus(2, 4),
}


def by_name(name: str) -> torch.Tensor:
    """Look a topology up by name; ``torusMxN`` and ``ringN`` are parsed."""
    if name in TOPOLOGIES:
        return TOPOLOGIES[name]()
    if name.startswith("torus") and "x" in name:
        m, n = name[5:].split("x")
        return torus(int(m), int(n))
    if name.startswith("ring"):
        return ring(int(name[4:]))
    raise KeyError(f"unknown topology {name!r}")
