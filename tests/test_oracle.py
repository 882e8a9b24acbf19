"""The CPU oracle (plain-C restatement) pinned against the reference's own outputs: the golden
vectors under tests/golden/ (made by the unmodified reference) and, where the compiled reference is
available, live runs of it on more seeded cases."""
import types

import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import synth

MAN = common.manifest()
SCHED = [k for k, v in MAN.items() if "kind" in v and "chain" not in v]
OUTS = [k for k, v in MAN.items() if "chain" in v]
SDDMM = [k for k, v in MAN.items() if "kq" in v]
NORMS = [k for k in MAN if k.startswith("gcn_norm_")]


def _oracle_schedule(oracle, kind, a, prm):
    if kind == 1:
        return oracle.inspect_fixed(a[0], a[1], prm["threads"], prm["iter_per_part"])
    return oracle.inspect_variable(kind, a[0], a[1], prm["threads"], prm["tile_m"], prm["bcol"], prm.get("ccol", 0))


def _golden_schedule(name):
    g = common.golden(name)
    return types.SimpleNamespace(n1=int(g["n1"]), ptr1=g["ptr1"], ptr2=g["ptr2"], id=g["id"], type=g["type"],
                                 ker_begin=g["ker"] if bool(g["has_ker"]) else None, stats=g["stats"])


@pytest.mark.parametrize("name", SCHED)
def test_oracle_schedule_matches_golden(oracle, name):
    case = MAN[name]
    a = common.matrix(case["matrix"])
    s = _oracle_schedule(oracle, case["kind"], a, case["params"])
    g = _golden_schedule(name)
    assert common.same_schedule(s, g)
    np.testing.assert_array_equal(s.stats[:5], g.stats)


@pytest.mark.parametrize("name", OUTS)
def test_oracle_output_matches_golden(oracle, name):
    case = MAN[name]
    a = common.matrix(case["matrix"])
    m = len(a[0]) - 1
    s = _oracle_schedule(oracle, case["kind"], a, case["params"])
    g = common.golden(name)
    want = g["D"]
    rows = g["rows"] if "rows" in g else np.arange(m)   # the larger fixtures keep every 4th row and two sums
    if case["chain"] == "spmm_spmm":
        c = synth.uniform(3, (m, case["dims"]["n"]))
        d, _ = oracle.spmm_spmm(a, a, c, s)
        # both chain FMAs in CSR order: bit-identical to the AVX2 reference kernel
        np.testing.assert_array_equal(d[rows], want)
    else:
        b = synth.uniform(2, (m, case["dims"]["k"]))
        w = synth.uniform(3, (case["dims"]["k"], case["dims"]["n"]))
        d, _ = oracle.gemm_spmm(a, b, w, s)
        common.assert_close(d[rows], want, name)
        d2, _ = oracle.gemm_spmm(a, b, np.ascontiguousarray(w.T), s, w_transposed=True)
        np.testing.assert_array_equal(d, d2)
    if "total" in g:
        common.assert_sums(d, g, name)


@pytest.mark.parametrize("name", SDDMM)
def test_oracle_sddmm_matches_the_reference_function(oracle, name):
    """S = A .* (Q K^T) against the values the reference's own sddmm_cpu (codegen/triton/sddmm.py:173-184)
    produced on the same seeded inputs; the reference checks its GPU kernels against that function with
    atol 1e-6 (ibid. :265-306)."""
    case = MAN[name]
    spec, kq = case["matrix"], case["kq"]
    a = synth.rmat_pattern(spec[1], spec[2], spec[3])
    n = len(a[0]) - 1
    q, k = synth.normal(2, (n, kq), 0.125), synth.normal(3, (n, kq), 0.125)
    v = synth.normal(4, (n, 32), 0.125)
    _, s = oracle.sddmm_spmm(a, q, k, v, want_s=True)
    want = common.golden(name)["S"]
    common.assert_close(s, want, name)
    assert np.abs(s - want).max() <= 1e-6


@pytest.mark.parametrize("name", NORMS)
def test_gcn_normalisation_matches_the_reference(name):
    """The values of synth.rmat_gcn are, bit for bit, what the reference's normalizeAdjacencyMatrix
    (fusion/gcn/SingleLayer/GCN_Single_Layer_SP_Demo_Utils.h:40-53) makes of all-ones values."""
    spec = MAN[name]["matrix"]
    ap, ai, ax = synth.rmat_gcn(spec[1], spec[2], spec[3])
    np.testing.assert_array_equal(ax, common.golden(name)["Ax"])


def test_gcn_normalisation_against_the_live_reference(ref):
    ap, ai, ax = synth.rmat_gcn(12, 900, 11)
    np.testing.assert_array_equal(ref.normalize_adjacency(ap, ai, np.ones(len(ai))).astype(np.float32), ax)


@pytest.mark.parametrize("dims,threads", [((97,), 2), ((33, 21), 3), ((9, 8, 7), 2), ((256, 256), 8)])
def test_oracle_vs_live_reference_schedules(oracle, ref, dims, threads):
    a = synth.laplacian(dims)
    m = len(a[0]) - 1
    for ipp in (16, 100, 2048):
        if m // ipp > 4096:
            continue  # the reference allocates partitions^2 bits for its DAG
        assert common.same_schedule(ref.inspect(1, a[0], a[1], threads, iter_per_part=ipp),
                                    oracle.inspect_fixed(a[0], a[1], threads, ipp))
    for tile_m in (20000, 100000, 1250000):
        for bcol in (32, 64):
            if m >= 64 * threads:
                s = oracle.inspect_variable(2, a[0], a[1], threads, tile_m, bcol)
                if s is not None:
                    assert common.same_schedule(ref.inspect(2, a[0], a[1], threads, tile_m=tile_m, bcol=bcol), s)
            if (tile_m // 4 - bcol * 48) // (bcol + 48) > 0:
                assert common.same_schedule(ref.inspect(3, a[0], a[1], threads, tile_m=tile_m, bcol=bcol, ccol=48),
                                            oracle.inspect_variable(3, a[0], a[1], threads, tile_m, bcol, 48))
            assert common.same_schedule(ref.inspect(4, a[0], a[1], threads, tile_m=tile_m, bcol=bcol),
                                        oracle.inspect_variable(4, a[0], a[1], threads, tile_m, bcol))


def test_known_answers_of_the_reference(oracle):
    """Facts about the reference inspectors on the 2-D 256x256 and 1-D operators."""
    a = synth.laplacian((256, 256))
    s = oracle.inspect_variable(3, a[0], a[1], 8, 1250000, 64, 64)
    assert list(s.ptr1) == [0, 54, 77] and s.stats[0] == 38400 and abs(s.stats[2] - 1213.63) < 0.01
    s = oracle.inspect_variable(3, a[0], a[1], 8, 300000, 64, 64)
    assert list(s.ptr1) == [0, 236, 491] and s.stats[0] == 43
    s = oracle.inspect_fixed(a[0], a[1], 8, 2048)
    assert list(s.ptr1) == [0, 32, 64] and s.stats[0] == 49664
    a = synth.laplacian((1000,))
    s = oracle.inspect_fixed(a[0], a[1], 4, 64)
    assert list(s.ptr1) == [0, 15, 30] and s.stats[0] == 972 and list(s.ker_begin[:2]) == [67, 133]
    c = np.ones((1000, 32), np.float32)
    d, _ = oracle.spmm_spmm(a, a, c, s)
    assert d.sum() == 64 and (d[0] == 2).all() and (d[1] == -1).all()


def test_oracle_executors_vs_live_reference(oracle, ref):
    a = synth.rmat_gcn(9, 700, 7)
    m = 700
    s = oracle.inspect_fixed(a[0], a[1], 3, 50)
    c = synth.uniform(3, (m, 64))
    d_ref, _ = ref.spmm_spmm(a, a, c, s, threads=3, variant=1)
    d_sc, _ = ref.spmm_spmm(a, a, c, s, threads=3, variant=0)
    d_orc, _ = oracle.spmm_spmm(a, a, c, s)
    np.testing.assert_array_equal(d_ref, d_orc)
    common.assert_close(d_sc, d_ref, "scalar vs AVX2 reference")
    common.assert_close(d_orc, oracle.chain_f64(a, c, b_sparse=a), "oracle vs fp64")
    b = synth.uniform(2, (m, 40))
    w = synth.uniform(4, (40, 96))
    g_ref, _ = ref.gemm_spmm(a, b, w, s, threads=3, variant=1)
    g_orc, _ = oracle.gemm_spmm(a, b, w, s)
    common.assert_close(g_orc, g_ref, "GeMM-SpMM oracle vs reference")
    common.assert_close(g_orc, oracle.chain_f64(a, w, b_dense=b), "GeMM-SpMM oracle vs fp64")


def test_composed_chains_agree_with_fp64(oracle):
    """SDDMM-SpMM and the 2-layer GCN as whole chains have no reference executor -- their parts do (sddmm_cpu,
    the CSR SpMM, the fused GCN layer, the adjacency normalisation; pinned above) -- so the composed fp32
    restatement is also cross-checked against an fp64 one."""
    a = synth.rmat_pattern(4, 600, 9)
    q, k = synth.normal(2, (600, 64), 0.125), synth.normal(3, (600, 64), 0.125)
    v = synth.normal(4, (600, 128), 0.125)
    d, s = oracle.sddmm_spmm(a, q, k, v, want_s=True)
    common.assert_close(d, oracle.sddmm_spmm_f64(a, q, k, v), "SDDMM-SpMM fp32 vs fp64")
    rows = np.repeat(np.arange(600), np.diff(a[0]))
    s64 = (q[rows].astype(np.float64) * k[a[1]].astype(np.float64)).sum(1) * a[2]
    common.assert_close(s, s64, "SDDMM values")
    g = synth.rmat_gcn(6, 500, 10)
    x = synth.normal(2, (500, 100))
    w1, w2 = synth.glorot(3, 256, 100), synth.glorot(4, 47, 256)
    out = oracle.gcn2(g, x, w1, w2)
    import scipy.sparse as sp
    A = sp.csr_matrix((g[2].astype(np.float64), g[1], g[0]), shape=(500, 500))
    h = np.maximum(A @ (x.astype(np.float64) @ w1.T.astype(np.float64)), 0)
    common.assert_close(out, A @ (h @ w2.T.astype(np.float64)), "GCN fp32 vs fp64")
