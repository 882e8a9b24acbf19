"""The sweep driver over matrix files (tile_fusion_b200/sweep.py), end to end on two small files."""
import csv

import numpy as np
import pytest
import scipy.io
import scipy.sparse as sp

from tile_fusion_b200 import sweep, synth

pytestmark = pytest.mark.gpu


def test_sweep_over_a_folder(built_lib, tmp_path):
    a = synth.laplacian((10, 8, 6))
    n = len(a[0]) - 1
    scipy.io.mmwrite(str(tmp_path / "lap.mtx"), sp.csr_matrix((a[2], a[1], a[0]), shape=(n, n)))
    g = synth.rmat_pattern(3, 700, 6)
    (tmp_path / "graph.smtx").write_text(f"700, 700, {len(g[1])}\n" + " ".join(map(str, g[0])) + "\n" + " ".join(map(str, g[1])) + "\n")
    (tmp_path / "list.txt").write_text("lap.mtx\ngraph.smtx\nmissing.mtx\n")
    for chain in ("spmm_spmm", "gemm_spmm"):
        out = tmp_path / f"{chain}.csv"
        rc = sweep.main(["--folder", str(tmp_path), "--list", str(tmp_path / "list.txt"), "--chain", chain, "--bcols", "32,64",
                         "--k", "16", "--trials", "3", "--out", str(out), "--check"])
        assert rc == 0
        rows = list(csv.DictReader(open(out)))
        assert len(rows) == 6
        good = [r for r in rows if not r["check"].startswith("error")]
        assert len(good) == 4 and all(float(r["check"]) <= 1e-5 for r in good)
        assert {r["matrix"] for r in good} == {"lap.mtx", "graph.smtx"}
        assert all(r["check"].startswith("error") for r in rows if r["matrix"] == "missing.mtx")
        assert all(float(r["gflops"]) > 0 and int(r["nnz"]) > 0 for r in good)
