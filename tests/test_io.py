"""Matrix ingestion (tile_fusion_b200/csrc/io.cpp): Matrix Market and DLMC .smtx files, the formats the reference's
drivers read (fusion/src/Fusion_Utils.cpp:205-283).  No GPU needed."""
import numpy as np
import pytest
import scipy.io
import scipy.sparse as sp

from tile_fusion_b200 import api
from tile_fusion_b200._lib import TileFusionError


def _same(A: api.CSRMatrix, S):
    S = sp.csr_matrix(S)
    S.sum_duplicates()
    S.sort_indices()
    assert (A.M, A.N) == S.shape
    np.testing.assert_array_equal(A.Ap, S.indptr)
    np.testing.assert_array_equal(A.Ai, S.indices)
    np.testing.assert_array_equal(A.Ax, S.data.astype(np.float32))


def test_matrix_market_general_and_symmetric(built_lib, tmp_path):
    rng = np.random.default_rng(3)
    S = sp.random(37, 29, density=0.12, random_state=5, format="coo", dtype=np.float64)
    S.data = np.round(S.data * 100) / 4
    scipy.io.mmwrite(str(tmp_path / "g.mtx"), S, comment="a general matrix")
    _same(api.read_matrix(tmp_path / "g.mtx"), S)
    L = sp.tril(sp.random(25, 25, density=0.2, random_state=7, dtype=np.float64)).tocoo()
    L.data = np.round(L.data * 64)
    full = L + sp.tril(L, -1).T
    scipy.io.mmwrite(str(tmp_path / "s.mtx"), full, symmetry="symmetric")
    _same(api.read_matrix(tmp_path / "s.mtx"), full)                      # the stored triangle is mirrored
    _same(api.read_matrix(tmp_path / "s.mtx", expand_symmetric=False), sp.tril(full))
    # pattern file with a duplicate entry and comment lines between header and sizes
    (tmp_path / "p.mtx").write_text("%%MatrixMarket matrix coordinate pattern general\n% one\n%two\n3 4 4\n1 1\n3 4\n2 2\n3 4\n")
    A = api.read_matrix(tmp_path / "p.mtx")
    _same(A, sp.coo_matrix(([1, 1, 2], ([0, 1, 2], [0, 1, 3])), shape=(3, 4)))
    del rng


def test_smtx(built_lib, tmp_path):
    S = sp.random(50, 40, density=0.1, random_state=11, format="csr")
    S.sort_indices()
    S.data[:] = 1
    text = f"{S.shape[0]}, {S.shape[1]}, {S.nnz}\n" + " ".join(map(str, S.indptr)) + "\n" + " ".join(map(str, S.indices)) + "\n"
    (tmp_path / "d.smtx").write_text(text)
    _same(api.read_matrix(tmp_path / "d.smtx"), S)


def test_dense_array_file(built_lib, tmp_path):
    x = np.arange(12, dtype=np.float64).reshape(4, 3) / 8
    scipy.io.mmwrite(str(tmp_path / "x.mtx"), x)
    np.testing.assert_array_equal(api.read_dense_mtx(tmp_path / "x.mtx"), x.astype(np.float32))


@pytest.mark.parametrize("name,text", [("missing.mtx", None), ("a.txt", "1 1 1\n"), ("bad.mtx", "hello\n"),
                                       ("short.mtx", "%%MatrixMarket matrix coordinate real general\n2 2 3\n1 1 1.0\n"),
                                       ("range.mtx", "%%MatrixMarket matrix coordinate real general\n2 2 1\n3 1 1.0\n"),
                                       ("ptr.smtx", "2, 2, 2\n0 1\n0 1\n")])
def test_bad_files_are_errors_not_exits(built_lib, tmp_path, name, text):
    if text is not None:
        (tmp_path / name).write_text(text)
    with pytest.raises(TileFusionError):
        api.read_matrix(tmp_path / name)
