"""CPU emulation of the persistent executor's item protocol (test helper).

Walks an item list the way the CTAs do -- up to `window` tickets in flight, any ready one may run
next -- with the same ring addressing and the same two watermarks, and computes D with numpy.  It
checks that no item can deadlock and that no ring slot is read before it is written or after it is
overwritten, which is what the `need` fields have to guarantee.
"""
from __future__ import annotations

import numpy as np


def _spmm_rows(ap, ai, ax, rows, dense_row):
    out = []
    for r in rows:
        acc = 0.0
        for p in range(ap[r], ap[r + 1]):
            acc = acc + np.float64(ax[p]) * dense_row(ai[p])
        out.append(acc)
    return out


def run_items(items, info, first, second, C, n_cols, m_local, window=16, seed=0, produce=None, ptile=None,
              ctile=None):
    """first/second: (ap, ai, ax).  produce(r) overrides the producer row (dense producer).
    ptile / ctile: (row_ptr, rows, halo_ptr, halo) of the gather tiles when items of kind 4 / 5 occur.
    Returns D (float64) and the intermediate tag array used for the checks."""
    rng = np.random.default_rng(seed)
    ring = info["ring_rows"]
    rows_alloc = info["intermediate_rows"]
    T = np.full((rows_alloc, n_cols), np.nan)
    tag = np.full(rows_alloc, -1, dtype=np.int64)  # which global row a slot currently holds
    D = np.full((m_local, n_cols), np.nan)
    n_prod, n_cons = info["producer_blocks"], info["consumer_blocks"]
    pdone = np.zeros(n_prod + 1, bool)
    cdone = np.zeros(n_cons + 1, bool)
    pw = cw = 0
    nxt, active = 0, []
    begin, end = info["phase1_begin"], info["end"]
    order = list(range(begin, end))
    seg_left = {}  # segments of a cut row still to run; the row counts as produced after the last one
    for t in order:
        if items[t][0] == 6:
            seg_left[items[t][2]] = seg_left.get(items[t][2], 0) + 1
    while nxt < len(order) or active:
        while nxt < len(order) and len(active) < window:
            active.append(order[nxt]); nxt += 1
        ready = []
        for t in active:
            kind, block, rb, re, need, base = items[t][:6]
            wm = pw if kind in (1, 5, 7) else cw
            if need <= wm:
                ready.append(t)
        assert ready, "deadlock: no in-flight item is ready"
        t = ready[rng.integers(len(ready))]
        active.remove(t)
        kind, block, rb, re, need, base = items[t][:6]
        if kind in (0, 4):
            rows = range(rb, re) if kind == 0 else ptile[1][ptile[0][rb]:ptile[0][rb + 1]]
            if kind == 4:  # a tiled producer may only touch the source rows it staged
                staged = set(ptile[3][ptile[2][rb]:ptile[2][rb + 1]].tolist())
                for r in rows:
                    assert set(first[1][first[0][r]:first[0][r + 1]].tolist()) <= staged
            for r in rows:
                slot = r
                if ring:
                    slot = r - base
                    assert 0 <= slot < 2 * ring, "producer row outside the item's ring window"
                    if slot >= ring:
                        slot -= ring
                if produce is not None:
                    T[slot] = produce(r)
                else:
                    acc = np.zeros(n_cols)
                    for p in range(first[0][r], first[0][r + 1]):
                        acc += np.float64(first[2][p]) * C[first[1][p]]
                    T[slot] = acc
                tag[slot] = r
            pdone[block] = True
            while pw < n_prod and pdone[pw]:
                pw += 1
        elif kind == 6:  # nonzeros [re, base) of row rb, added to T[rb]
            assert not ring
            acc = np.zeros(n_cols) if np.isnan(T[rb]).any() else T[rb].copy()
            for p in range(re, base):
                acc += np.float64(first[2][p]) * C[first[1][p]]
            T[rb] = acc
            seg_left[rb] -= 1
            if seg_left[rb] == 0:
                tag[rb] = rb
            pdone[block] = True
            while pw < n_prod and pdone[pw]:
                pw += 1
        elif kind == 7:  # nonzeros [re, base) of row rb, added to D[rb]
            assert not ring
            acc = np.zeros(n_cols) if np.isnan(D[rb]).any() else D[rb].copy()
            for p in range(re, base):
                col = second[1][p]
                if col < m_local:
                    assert tag[col] == col, "intermediate row read before it was produced"
                acc += np.float64(second[2][p]) * T[col]
            D[rb] = acc
        elif kind in (1, 5):
            rows = range(rb, re) if kind == 1 else ctile[1][ctile[0][rb]:ctile[0][rb + 1]]
            if kind == 5:
                staged = set(ctile[3][ctile[2][rb]:ctile[2][rb + 1]].tolist())
                for r in rows:
                    assert set(second[1][second[0][r]:second[0][r + 1]].tolist()) <= staged
            for r in rows:
                acc = np.zeros(n_cols)
                for p in range(second[0][r], second[0][r + 1]):
                    col = second[1][p]
                    if ring:
                        if col >= m_local:
                            slot = ring + (col - m_local)
                        else:
                            slot = col - base
                            assert 0 <= slot < 2 * ring, "column outside the item's ring window"
                            if slot >= ring:
                                slot -= ring
                            assert tag[slot] == col, f"ring slot holds row {tag[slot]}, wanted {col}"
                    else:
                        slot = col
                        if col < m_local:
                            assert tag[slot] == col, "intermediate row read before it was produced"
                    acc += np.float64(second[2][p]) * T[slot]
                D[r] = acc
            if ring:
                cdone[block] = True
                while cw < n_cons and cdone[cw]:
                    cw += 1
    return D, T
