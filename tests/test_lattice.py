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
