"""Row-block partition of a fused chain over ranks (one process per GPU).

The reference runs on one shared-memory host; the partition is this library's own.  Rule
(deterministic, so every rank derives the same arrays):

* rank g owns the contiguous rows [bounds[g], bounds[g+1]) of A, of the intermediate T and of D;
* its halo is the sorted list of column ids of its rows of A that fall outside its own range;
  the rows of T with those ids arrive from their owners and are stored after the local rows;
* its boundary is the sorted list of its own rows that appear in some other rank's halo; they
  are produced first (phase 0) into a send buffer laid out in that order.

Only halo rows of T travel; there is no other collective on the data path.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


def row_bounds(ap: np.ndarray | None, n_rows: int, world: int, by: str = "rows") -> np.ndarray:
    """Partition boundaries: equal rows ("rows") or equal nonzeros ("nnz", needs the global Ap)."""
    if by == "rows" or ap is None:
        base, rem = divmod(n_rows, world)
        sizes = np.full(world, base, dtype=np.int64)
        sizes[:rem] += 1
        return np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    target = np.arange(1, world) * (int(ap[-1]) / world)
    cuts = np.searchsorted(ap, target, side="left")
    return np.concatenate([[0], cuts, [n_rows]]).astype(np.int64)


@dataclass
class Segment:
    peer: int
    start: int   # first row inside the send / halo buffer
    count: int
    index: np.ndarray | None = None  # send side only: rows of the send buffer to gather when not contiguous


@dataclass
class RankLayout:
    rank: int
    world: int
    bounds: np.ndarray          # world + 1 global row boundaries
    halo_ids: np.ndarray        # sorted global ids of the T rows received
    boundary_rows: np.ndarray   # sorted LOCAL ids of the T rows sent
    recv: list = field(default_factory=list)   # Segment per peer, into the halo buffer
    send: list = field(default_factory=list)   # Segment per peer, out of the send buffer

    @property
    def r0(self):
        return int(self.bounds[self.rank])

    @property
    def r1(self):
        return int(self.bounds[self.rank + 1])

    @property
    def m(self):
        return self.r1 - self.r0


def halo_of(ai_global: np.ndarray, r0: int, r1: int) -> np.ndarray:
    """Sorted unique column ids outside [r0, r1)."""
    out = ai_global[(ai_global < r0) | (ai_global >= r1)]
    return np.unique(out).astype(np.int64)


def make_layout(rank: int, bounds: np.ndarray, halos: list) -> RankLayout:
    """halos[g] = halo_of(rows of rank g) for every rank g (all ranks hold the same list)."""
    world = len(bounds) - 1
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    mine = halos[rank]
    lay = RankLayout(rank, world, np.asarray(bounds, dtype=np.int64), mine, np.zeros(0, np.int64))
    owner = np.searchsorted(bounds, mine, side="right") - 1
    pos = 0
    for p in range(world):
        cnt = int((owner == p).sum())
        if cnt:
            lay.recv.append(Segment(p, pos, cnt))
            pos += cnt
    wanted = {}
    for g in range(world):
        if g == rank:
            continue
        h = halos[g]
        sel = h[(h >= r0) & (h < r1)] - r0
        if len(sel):
            wanted[g] = sel
    if wanted:
        lay.boundary_rows = np.unique(np.concatenate(list(wanted.values()))).astype(np.int64)
    for g, sel in wanted.items():
        idx = np.searchsorted(lay.boundary_rows, sel)
        contiguous = len(idx) == 0 or (idx[-1] - idx[0] + 1 == len(idx))
        lay.send.append(Segment(g, int(idx[0]), len(idx), None if contiguous else idx.astype(np.int64)))
    return lay


def localize_columns(ai_global: np.ndarray, lay: RankLayout) -> np.ndarray:
    """Column ids of the rank's rows of A in the executor's numbering: own rows -> [0, m),
    halo rows -> m + position in halo_ids."""
    ai = np.asarray(ai_global, dtype=np.int64)
    local = (ai >= lay.r0) & (ai < lay.r1)
    out = np.empty(ai.shape, dtype=np.int64)
    out[local] = ai[local] - lay.r0
    out[~local] = lay.m + np.searchsorted(lay.halo_ids, ai[~local])
    return out.astype(np.int32)


def compact_columns(ai_global: np.ndarray):
    """For the first operator of SpMM-SpMM: the sorted global ids of the rows of C the rank's rows
    touch (own + ghost) and the column ids renumbered into that list."""
    ids = np.unique(ai_global).astype(np.int64)
    return ids, np.searchsorted(ids, ai_global).astype(np.int32)
