"""Host logic of the stream planner, checked by emulating the executor's protocol on the CPU."""
import numpy as np
import pytest

from tile_fusion_b200 import api, synth
from tests.emulate import run_items


def _csr(t):
    n = len(t[0]) - 1
    return api.CSRMatrix(n, n, *t)


def _dense_chain(t, C):
    import scipy.sparse as sp
    n = len(t[0]) - 1
    A = sp.csr_matrix((t[2].astype(np.float64), t[1], t[0]), shape=(n, n))
    return A @ (A @ C.astype(np.float64))


@pytest.mark.parametrize("dims,rb,slack,ring_bytes,window", [
    ((16, 16), 8, 2, 1 << 30, 8),      # ring active
    ((6, 6, 6), 4, 3, 1 << 30, 12),    # 3-D stencil, ring active
    ((16, 16), 8, 2, -1, 8),           # ring off
    ((40,), 4, 1, 1 << 30, 5),
])
def test_stream_plan_emulation(built_lib, dims, rb, slack, ring_bytes, window):
    t = synth.laplacian(dims)
    A = _csr(t)
    n, nc = A.M, 3
    C = synth.uniform(7, (n, nc)).astype(np.float64)
    items, info = api.plan_preview(A, n_cols=nc, rows_per_block=rb, slack_blocks=slack, ring_bytes=ring_bytes,
                                   resident_ctas=window, tile_slots=-1)
    if ring_bytes > 0:
        assert 0 < info["ring_rows"] < n, info
    else:
        assert info["ring_rows"] == 0
    assert info["items"] == info["producer_blocks"] + info["consumer_blocks"]
    want = _dense_chain(t, C)
    for seed in range(3):
        D, _ = run_items(items, info, t, t, C, nc, n, window=window, seed=seed)
        np.testing.assert_allclose(D, want, rtol=1e-12, atol=1e-12)


def test_stream_plan_random_pattern(built_lib):
    """Unstructured pattern: windows span everything, so the planner must fall back to a full intermediate."""
    ap, ai, ax = synth.rmat_gcn(3, 200, 6)
    A = api.CSRMatrix(200, 200, ap, ai, ax)
    C = synth.uniform(5, (200, 2)).astype(np.float64)
    items, info = api.plan_preview(A, n_cols=2, rows_per_block=8, slack_blocks=2, resident_ctas=8)
    D, _ = run_items(items, info, (ap, ai, ax), (ap, ai, ax), C, 2, 200, window=8, seed=1)
    np.testing.assert_allclose(D, _dense_chain((ap, ai, ax), C), rtol=1e-10, atol=1e-12)


def test_heavy_rows_get_their_own_block(built_lib):
    n = 300
    rows = [np.arange(n, dtype=np.int32) if r == 17 else np.array([r], np.int32) for r in range(n)]
    ap = np.zeros(n + 1, np.int32)
    ap[1:] = np.cumsum([len(r) for r in rows])
    ai = np.concatenate(rows)
    ax = np.ones(len(ai), np.float32)
    A = api.CSRMatrix(n, n, ap, ai, ax)
    items, info = api.plan_preview(A, n_cols=4, rows_per_block=8, slack_blocks=1, tile_slots=-1)
    cons = items[items[:, 0] == 1]
    blk = cons[(cons[:, 2] <= 17) & (cons[:, 3] > 17)][0]
    assert blk[3] - blk[2] == 1  # 300 nnz > 8*32: the heavy row stands alone
    assert cons[:, 3].max() == n and (np.diff(cons[:, 2]) > 0).all()


def _hub_matrix(n, hub_rows, seed=3):
    """Diagonal plus a few rows that touch (almost) every column."""
    rows = []
    for r in range(n):
        if r in hub_rows:
            rows.append(np.arange(hub_rows[r], dtype=np.int32))
        else:
            rows.append(np.unique(np.array([r, (r * 7 + 1) % n], np.int32)))
    ap = np.zeros(n + 1, np.int32)
    ap[1:] = np.cumsum([len(r) for r in rows])
    ai = np.concatenate(rows)
    ax = (synth.uniform(seed, (len(ai),)) - 0.5).astype(np.float32)
    return ap, ai, ax


@pytest.mark.parametrize("mode", [api.MODE_STREAM, api.MODE_UNFUSED])
def test_hub_rows_are_cut_into_segments(built_lib, mode):
    n = 9500
    t = _hub_matrix(n, {17: 9300, 4000: 5000, 9499: 600})
    A = api.CSRMatrix(n, n, *t)
    items, info = api.plan_preview(A, n_cols=2, rows_per_block=64, slack_blocks=2, resident_ctas=12, tile_slots=-1,
                                   mode=mode)
    assert info["ring_rows"] == 0
    for kind, n17, n4000 in ((6, 3, 2), (7, 3, 2)):
        seg = items[items[:, 0] == kind]
        assert (seg[:, 2] == 17).sum() == n17 and (seg[:, 2] == 4000).sum() == n4000
        assert ((seg[:, 5] - seg[:, 3]) <= 4096).all() and ((seg[:, 5] - seg[:, 3]) > 0).all()
        # the segments of a row cover its nonzeros once
        s17 = seg[seg[:, 2] == 17]
        assert s17[0, 3] == t[0][17] and s17[-1, 5] == t[0][18] and (s17[1:, 3] == s17[:-1, 5]).all()
    whole = items[(items[:, 0] == 1) & (items[:, 2] == 9499)]
    assert len(whole) == 1 and whole[0, 3] == n  # 600 nonzeros: alone in its block, not cut
    C = synth.uniform(5, (n, 2)).astype(np.float64)
    want = _dense_chain(t, C)
    for seed in range(2):
        D, _ = run_items(items, info, t, t, C, 2, n, window=12, seed=seed)
        np.testing.assert_allclose(D, want, rtol=1e-10, atol=1e-10)


def test_unfused_mode_lists_all_producers_first(built_lib):
    t = synth.laplacian((12, 12))
    A = _csr(t)
    items, info = api.plan_preview(A, n_cols=8, rows_per_block=8, mode=api.MODE_UNFUSED, tile_slots=-1)
    k = info["producer_blocks"]
    assert (items[:k, 0] == 0).all() and (items[k:, 0] == 1).all() and info["ring_rows"] == 0


def test_halo_plan_defers_halo_consumers(built_lib):
    """Multi-GPU layout: A is m x (m + halo); consumers that read halo rows go to phase 2."""
    t = synth.laplacian((8, 8, 4))           # global
    n = 8 * 8 * 4
    m, plane = 128, 64                        # this rank owns rows [64, 192): planes 1 and 2
    r0 = 64
    ap, ai, ax = t
    rows = range(r0, r0 + m)
    cols, vals, ptr = [], [], [0]
    halo_ids = sorted({int(c) for r in rows for c in ai[ap[r]:ap[r + 1]] if not (r0 <= c < r0 + m)})
    hmap = {g: m + i for i, g in enumerate(halo_ids)}
    for r in rows:
        for p in range(ap[r], ap[r + 1]):
            c = int(ai[p])
            cols.append(c - r0 if r0 <= c < r0 + m else hmap[c]); vals.append(ax[p])
        ptr.append(len(cols))
    A = api.CSRMatrix(m, m + len(halo_ids), np.array(ptr, np.int32), np.array(cols, np.int32),
                      np.array(vals, np.float32))
    boundary = np.array(list(range(0, plane)) + list(range(m - plane, m)), np.int32)
    items, info = api.plan_preview(A, producer_is_gemm=True, n_cols=4, rows_per_block=16, slack_blocks=1,
                                   halo_rows=len(halo_ids), boundary_rows=boundary, tile_slots=-1)
    assert info["ring_rows"] == 0 and info["intermediate_rows"] == m + len(halo_ids)
    p1 = items[info["phase1_begin"]:info["phase2_begin"]]
    p2 = items[info["phase2_begin"]:info["end"]]
    assert (p2[:, 0] == 1).all() and len(p2) == 2 * plane // 16  # first and last plane read halo rows
    assert (p1[:, 0] == 0).sum() == m // 16 and (p1[:, 0] == 1).sum() == 0  # 2 planes: every consumer touches a halo


@pytest.mark.parametrize("dims,slots,max_bz,ring_bytes,slack,window", [
    ((24, 20, 12), 200, 2, 1 << 30, 3, 10),   # 3-D bricks through a ring
    ((24, 20, 12), 300, 4, -1, 3, 10),        # 3-D bricks, full intermediate
    ((40, 36), 120, 1, 1 << 30, 2, 8),        # 2-D bricks through a ring
    ((500,), 80, 1, 1 << 30, 2, 6),           # 1-D
])
def test_tiled_plan_emulation(built_lib, dims, slots, max_bz, ring_bytes, slack, window):
    """Gather tiles: every tile stages all the source rows its rows name, every row is in exactly one
    tile, and the ticket order / ring waits hold under random interleavings."""
    t = synth.laplacian(dims)
    A = _csr(t)
    n, nc = A.M, 4
    til = api.tiling_preview(A, tile_slots=slots, tile_max_bz=max_bz)
    assert til is not None
    row_ptr, rows, halo_ptr, halo, tinfo = til
    assert sorted(rows.tolist()) == list(range(n))
    assert (np.diff(halo_ptr) <= slots).all() and tinfo["reuse"] >= 2.0
    items, info = api.plan_preview(A, n_cols=nc, slack_blocks=slack, ring_bytes=ring_bytes, resident_ctas=window,
                                   tile_slots=slots, tile_max_bz=max_bz)
    assert set(items[:, 0].tolist()) == {4, 5}
    if ring_bytes > 0:
        assert 0 < info["ring_rows"] < n, info
    C = synth.uniform(7, (n, nc)).astype(np.float64)
    want = _dense_chain(t, C)
    for seed in range(2):
        D, _ = run_items(items, info, t, t, C, nc, n, window=window, seed=seed, ptile=til[:4], ctile=til[:4])
        np.testing.assert_allclose(D, want, rtol=1e-12, atol=1e-12)


def test_tiling_declined_without_structure(built_lib):
    # (a graph this sparse and this large reuses a staged row less than twice, whatever the tile)
    g = synth.rmat_gcn(3, 20000, 6)
    assert api.tiling_preview(api.CSRMatrix(20000, 20000, *g)) is None
    items, info = api.plan_preview(api.CSRMatrix(20000, 20000, *g), n_cols=32)
    assert set(items[:, 0].tolist()) == {0, 1}
