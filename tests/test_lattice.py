"""Host side of the plane-marching executor: recognising an operator as a star stencil on a 3-D grid
(tile_fusion_b200/csrc/lattice.cpp) and its work list.  No GPU needed."""
import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import api, synth


def _csr(t, ncols=None):
    n = len(t[0]) - 1
    return api.CSRMatrix(n, ncols or n, *t)


def _rebuild(r, shift=0):
    """CSR triplets (row, col, value) of the operator that a class table stands for."""
    nx, ny, nz = r["nx"], r["ny"], r["nz"]
    offs = [-nx * ny, -nx, -1, 0, 1, nx, nx * ny]
    out = {}
    for z in range(nz):
        for y in range(ny):
            for x in range(nx):
                w = int(r["patch_cls"][z, y // 2, x // 2])
                cls = (w >> (8 * (2 * (y & 1) + (x & 1)))) & 255
                row = (z * ny + y) * nx + x
                for k, o in enumerate(offs):
                    v = r["dict"][cls, k]
                    if v != 0:
                        out[(row, row + o + shift)] = v
    return out


@pytest.mark.parametrize("dims", [(6, 5, 4), (14, 14, 14), (8, 4, 3)])
def test_class_table_is_the_operator(built_lib, dims):
    a = synth.laplacian(dims)
    # make the values row dependent so that several coefficient classes exist beyond the boundary ones
    rows = np.repeat(np.arange(len(a[0]) - 1), np.diff(a[0]))
    ax = (a[2] * (1.0 + (rows % 2))).astype(np.float32)
    r = api.lattice_preview(_csr((a[0], a[1], ax)))
    assert r is not None and (r["nx"], r["ny"], r["nz"]) == dims
    assert np.all(r["dict"][-1] == 0)              # the last class is the all-zero vector
    got = _rebuild(r)
    want = {(int(i), int(j)): float(v) for i, j, v in zip(rows, a[1], ax)}
    assert got == want
    # class 0 is the most frequent one
    counts = np.bincount(r["patch_cls"].view(np.uint8).ravel(), minlength=r["classes"] + 1)
    assert counts[0] == counts[:r["classes"]].max()


def test_declined_patterns(built_lib):
    assert api.lattice_preview(_csr(synth.rmat_gcn(7, 3000, 14))) is None       # a graph
    assert api.lattice_preview(_csr(synth.laplacian((40, 33)))) is None          # two dimensions
    assert api.lattice_preview(_csr(synth.laplacian((9, 8, 7)))) is None         # odd x extent (rows are read in pairs)
    a = synth.laplacian((8, 6, 5))
    ai = a[1].copy()
    ai[a[0][100]] = 0                                                             # row 100 names a row that is no grid neighbour
    assert api.lattice_preview(_csr((a[0], ai, a[2]))) is None
    # more distinct coefficient vectors than the dictionary holds
    ax = (a[2] * (1.0 + np.repeat(np.arange(len(a[0]) - 1), np.diff(a[0])) % 97)).astype(np.float32)
    assert api.lattice_preview(_csr((a[0], a[1], ax))) is None


def test_shifted_columns_and_ghost_planes(built_lib):
    """Rows of one rank of a partitioned chain: its slab of a taller grid, columns renumbered so that the first
    ghost plane is column 0."""
    dims, n_cols = (8, 6, 12), 32
    plane = dims[0] * dims[1]
    r0, r1 = 3 * plane, 9 * plane
    ap, ai, ax = synth.laplacian_rows(dims, r0, r1)
    lo = int(ai.min())
    r = api.lattice_preview(api.CSRMatrix(r1 - r0, int(ai.max()) - lo + 1, ap, (ai - lo).astype(np.int32), ax), n_cols=n_cols)
    assert r is not None and (r["nx"], r["ny"], r["nz"]) == (8, 6, 6)
    assert (r["ghost_lo"], r["ghost_hi"]) == (1, 1)
    rows = np.repeat(np.arange(r1 - r0), np.diff(ap))
    assert _rebuild(r, shift=plane) == {(int(i), int(j)): float(v) for i, j, v in zip(rows, ai - lo, ax)}


@pytest.mark.parametrize("dims,n_cols,ctas", [((128, 128, 128), 128, 296), ((40, 34, 9), 100, 296), ((14, 14, 14), 4, 8)])
def test_items_cover_every_output_once(built_lib, dims, n_cols, ctas):
    r = api.lattice_preview(_csr(synth.laplacian(dims)), n_cols=n_cols, ctas=ctas)
    it = r["items"]
    nx, ny, nz = dims
    cover = np.zeros(((nx + 15) // 16, (ny + 7) // 8, nz, (n_cols + 15) // 16), np.int32)
    for x0, y0, zs, ze, c0, _ in it:
        assert x0 % 16 == 0 and y0 % 8 == 0 and c0 % 16 == 0 and 0 <= zs < ze <= nz
        cover[x0 // 16, y0 // 8, zs:ze, c0 // 16] += 1
    assert np.all(cover == 1)
    nch = (n_cols + 15) // 16
    if dims == (128, 128, 128):
        # the chunks of one tile are adjacent in the list (whole dense rows are read together)
        assert all(len({tuple(v[:4]) for v in it[i:i + nch]}) == 1 for i in range(0, len(it), nch))
    # CTAs take the items in list order as they become free; a piece of L planes takes L + 4 steps.  The slowest
    # CTA must not be slower than with equal cuts of every column (the best of 1 .. 16 cuts).
    import heapq
    free = [0] * ctas
    for x0, y0, zs, ze, c0, _ in it:
        heapq.heappush(free, heapq.heappop(free) + (ze - zs) + 4)
    columns = cover.shape[0] * cover.shape[1] * nch
    equal = min(-(-columns * s // ctas) * (-(-nz // s) + 4) for s in range(1, 17) if s == 1 or -(-nz // s) >= 8)
    assert max(free) <= equal
    if dims == (128, 128, 128):
        assert max(free) == 3 * 132 + 68       # three rounds of whole columns, then 296 pieces of at most 64 planes


def _apply_planes(r, c_planes, z):
    """One plane of (operator x operand) from the class table: out[y, x, :] = sum over the seven stencil points of
    dict[class(x, y, z)][k] * operand(point k), operand planes outside [0, nz) taken as zero."""
    nx, ny, nz = r["nx"], r["ny"], r["nz"]
    w = r["patch_cls"][z]
    ys, xs = np.meshgrid(np.arange(ny), np.arange(nx), indexing="ij")
    cls = (w[ys // 2, xs // 2] >> (8 * (2 * (ys & 1) + (xs & 1)))) & 255
    coef = r["dict"][cls].astype(np.float64)               # [ny, nx, 8]
    zero = np.zeros_like(c_planes[0])
    cur = c_planes[z]
    below = c_planes[z - 1] if z - 1 >= 0 else zero
    above = c_planes[z + 1] if z + 1 < nz else zero
    pad = np.pad(cur, ((1, 1), (1, 1), (0, 0)))
    parts = [below, pad[:-2, 1:-1], pad[1:-1, :-2], cur, pad[1:-1, 2:], pad[2:, 1:-1], above]
    return sum(coef[:, :, k, None] * p for k, p in enumerate(parts))


@pytest.mark.parametrize("dims,n_cols,ctas", [((8, 6, 10), 24, 5), ((18, 10, 7), 16, 296)])
def test_marching_recurrence_over_the_work_list(built_lib, dims, n_cols, ctas):
    """The plane-marching algorithm replayed on the host from what the library hands its kernel -- class words,
    dictionary, work items: every item marches its planes with the kernel's lead-in rule (two planes in front of the
    first output plane, none below plane 0), builds T one plane ahead of D and writes its tile's rows of D.  The
    union of the items must be A (A C)."""
    import scipy.sparse as sp
    a = synth.laplacian(dims)
    n = len(a[0]) - 1
    rows = np.repeat(np.arange(n), np.diff(a[0]))
    ax = (a[2] * (1.0 + 0.25 * (rows % 3))).astype(np.float32)
    r = api.lattice_preview(_csr((a[0], a[1], ax)), n_cols=n_cols, ctas=ctas)
    nx, ny, nz = dims
    c = synth.uniform(5, (n, n_cols)).astype(np.float64)
    c_planes = c.reshape(nz, ny, nx, n_cols)
    A = sp.csr_matrix((ax.astype(np.float64), a[1], a[0]), shape=(n, n))
    want = (A @ (A @ c)).reshape(nz, ny, nx, n_cols)
    got = np.full_like(want, np.nan)
    for x0, y0, zs, ze, c0, _ in r["items"]:
        cols = slice(c0, min(c0 + 16, n_cols))
        kfirst = zs - (0 if zs == 0 else 2)
        t_planes = {}
        for k in range(kfirst, ze + 2):          # plane C(k) arrives
            # T(k-1) is complete once C(k) is there; D(k-2) once T(k-1) is
            if 0 <= k - 1 < nz:
                t_planes[k - 1] = _apply_planes(r, c_planes, k - 1)[:, :, cols]
            z = k - 2
            if zs <= z < ze:
                t_full = np.zeros((nz, ny, nx, cols.stop - cols.start))
                for q in (z - 1, z, z + 1):
                    if 0 <= q < nz:
                        assert q in t_planes, (zs, ze, k, q)   # the lead-in planes were enough
                        t_full[q] = t_planes[q]
                d = _apply_planes(r, t_full, z)
                ty, tx = slice(y0, min(y0 + 8, ny)), slice(x0, min(x0 + 16, nx))
                assert np.all(np.isnan(got[z, ty, tx, cols]))     # every output is written once
                got[z, ty, tx, cols] = d[ty, tx]
    assert not np.isnan(got).any()
    np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-12)
