"""Reordered layouts and the RCM ordering (tile_fusion_b200/csrc/reorder.cpp).  No GPU needed."""
import numpy as np
import pytest
import scipy.sparse as sp

from tests import common
from tile_fusion_b200 import api, synth


@pytest.mark.parametrize("spec,kind,prm", [
    (("lap", (24, 24)), 3, dict(threads=2, tile_m=20000, b_cols=16, c_cols=32)),
    (("rmat_gcn", 5, 512, 6), 1, dict(threads=2, iter_per_partition=64)),
    (("lap", (12, 10, 9)), 2, dict(threads=2, tile_m=30000, b_cols=32)),
])
def test_layouts_match_the_reference(built_lib, ref, spec, kind, prm):
    """createUnfusedData / createReorderedAdj of the reference (compiled from its headers into oracle/_ref) on the
    schedule of its own inspector, against the library's builders on the library's (bit-identical) schedule."""
    a = common.matrix(spec)
    A = api.CSRMatrix(len(a[0]) - 1, len(a[0]) - 1, *a)
    s = api.inspector(A, prm["threads"], kind=kind, **{k: v for k, v in prm.items() if k != "threads"})
    (ufp, ufi, ufx), (rp, ri, rx, l2, mix) = ref.layouts(kind, a[0], a[1], a[2], prm["threads"],
                                                         iter_per_part=prm.get("iter_per_partition", 1), tile_m=prm.get("tile_m", 1),
                                                         bcol=prm.get("b_cols", 1), ccol=prm.get("c_cols", 1))
    got = api.unfused_csr(s, A)
    for g, w in zip(got, (ufp, ufi, ufx)):
        np.testing.assert_array_equal(g, w)
    got = api.reordered_adjacency(s, A)
    np.testing.assert_array_equal(got[0], rp)
    np.testing.assert_array_equal(got[1], ri)
    np.testing.assert_array_equal(got[2], rx)
    np.testing.assert_array_equal(got[3], l2)
    np.testing.assert_array_equal(got[4][2:], mix[2:])   # (the reference leaves the first pair as it initialised it: zeros)
    assert got[4][0] == 0 and got[4][1] == 0


def test_rcm_is_a_permutation_that_cuts_bandwidth(built_lib):
    rng = np.random.default_rng(0)
    a = synth.laplacian((30, 28))
    n = len(a[0]) - 1
    A = api.CSRMatrix(n, n, *a)
    shuffle = rng.permutation(n).astype(np.int32)
    B = api.permute(A, shuffle)                               # scatter the grid order
    S = sp.csr_matrix((a[2], a[1], a[0]), shape=(n, n))
    np.testing.assert_array_equal(sp.csr_matrix((B.Ax, B.Ai, B.Ap), shape=(n, n)).toarray(), S[shuffle][:, shuffle].toarray())
    perm = api.rcm_order(B)
    assert sorted(perm.tolist()) == list(range(n))
    C_ = api.permute(B, perm)

    def bandwidth(M):
        rows = np.repeat(np.arange(M.M), np.diff(M.Ap))
        return int(np.abs(M.Ai - rows).max())
    assert bandwidth(B) > 10 * bandwidth(C_)
    assert bandwidth(C_) <= 2 * 30                            # a grid of width 28-30 has bandwidth about its width
    assert np.all(np.diff(C_.Ai)[np.diff(np.repeat(np.arange(n), np.diff(C_.Ap))) == 0] > 0)   # columns sorted in every row
