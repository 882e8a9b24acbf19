"""The product inspector (C ABI) against the golden vectors, the oracle and the live reference:
schedule arrays must be bit-identical."""
import ctypes as C
import types

import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import _lib, api, synth

MAN = common.manifest()
SCHED = [k for k, v in MAN.items() if "kind" in v and "chain" not in v]


def _product_schedule(a, kind, prm):
    A = api.CSRMatrix(len(a[0]) - 1, len(a[0]) - 1, *a)
    return api.inspector(A, prm["threads"], kind=kind, iter_per_partition=prm.get("iter_per_part", 1),
                         tile_m=prm.get("tile_m", 1), b_cols=prm.get("bcol", 1), c_cols=prm.get("ccol", 1))


@pytest.mark.parametrize("name", SCHED)
def test_inspector_matches_golden(built_lib, name):
    case = MAN[name]
    g = common.golden(name)
    want = types.SimpleNamespace(n1=int(g["n1"]), ptr1=g["ptr1"], ptr2=g["ptr2"], id=g["id"], type=g["type"],
                                 ker_begin=g["ker"] if bool(g["has_ker"]) else None)
    s = _product_schedule(common.matrix(case["matrix"]), case["kind"], case["params"])
    assert common.same_schedule(s, want)
    np.testing.assert_array_equal(s.stats, g["stats"])


@pytest.mark.parametrize("dims,threads", [((500,), 2), ((40, 30), 3), ((12, 10, 9), 2), ((128, 128), 8),
                                          ((24, 24, 24), 4)])
def test_inspector_matches_oracle_sweep(built_lib, oracle, dims, threads):
    """The sweep of the reference's experiment driver (run_exp.sh mode 7), scaled down."""
    a = synth.laplacian(dims)
    m = len(a[0]) - 1
    for ipp in (16, 64, 256, 2048):
        prm = dict(threads=threads, iter_per_part=ipp)
        assert common.same_schedule(_product_schedule(a, 1, prm), oracle.inspect_fixed(a[0], a[1], threads, ipp))
    for tile_m in (60000, 100000, 500000, 1500000):
        for bcol, ccol in ((32, 32), (64, 128), (128, 47)):
            for kind in (2, 3, 4):
                want = oracle.inspect_variable(kind, a[0], a[1], threads, tile_m, bcol, ccol)
                prm = dict(threads=threads, tile_m=tile_m, bcol=bcol, ccol=ccol)
                if want is None:
                    with pytest.raises(api.TileFusionError):
                        _product_schedule(a, kind, prm)
                else:
                    got = _product_schedule(a, kind, prm)
                    assert common.same_schedule(got, want), (kind, tile_m, bcol, ccol)
                    np.testing.assert_array_equal(got.stats, want.stats[:5])


def test_inspector_on_skewed_graph(built_lib, oracle):
    a = synth.rmat_gcn(21, 5000, 12)
    for kind, prm in ((1, dict(threads=4, iter_per_part=100)), (2, dict(threads=4, tile_m=200000, bcol=64)),
                      (3, dict(threads=4, tile_m=400000, bcol=100, ccol=256)), (4, dict(threads=4, tile_m=200000, bcol=64))):
        want = (oracle.inspect_fixed(a[0], a[1], 4, 100) if kind == 1 else
                oracle.inspect_variable(kind, a[0], a[1], 4, prm["tile_m"], prm["bcol"], prm.get("ccol", 0)))
        assert common.same_schedule(_product_schedule(a, kind, prm), want)


def test_inspector_vs_live_reference(built_lib, ref):
    a = synth.laplacian((48, 40))
    for kind, prm in ((1, dict(threads=3, iter_per_part=128)), (2, dict(threads=3, tile_m=50000, bcol=32)),
                      (3, dict(threads=3, tile_m=90000, bcol=32, ccol=64)), (4, dict(threads=3, tile_m=50000, bcol=32))):
        want = ref.inspect(kind, a[0], a[1], prm["threads"], iter_per_part=prm.get("iter_per_part", 1),
                           tile_m=prm.get("tile_m", 1), bcol=prm.get("bcol", 1), ccol=prm.get("ccol", 1))
        assert common.same_schedule(_product_schedule(a, kind, prm), want)


def test_inspector_rejects_bad_input(built_lib):
    a = synth.laplacian((10, 10))
    A = api.CSRMatrix(100, 100, *a)
    with pytest.raises(api.TileFusionError):  # m < 2 * threads: the reference divides by zero
        api.inspector(A, 64, kind=api.INSPECT_VT_SPMM, tile_m=1000, b_cols=8)
    with pytest.raises(api.TileFusionError):  # cache budget below the dense operand
        api.inspector(A, 2, kind=api.INSPECT_VT_GEMM, tile_m=100, b_cols=64, c_cols=64)
    ai = a[1].copy()
    ai[[0, 1]] = ai[[1, 0]]  # unsorted row 0
    with pytest.raises(api.TileFusionError):
        api.inspector(api.CSRMatrix(100, 100, a[0], ai, a[2]), 2, kind=api.INSPECT_VT_SPMM, tile_m=10000, b_cols=8)
    bad = a[1].copy()
    bad[5] = 100
    with pytest.raises(api.TileFusionError):
        api.inspector(api.CSRMatrix(100, 100, a[0], bad, a[2]), 2)
    with pytest.raises(api.TileFusionError):
        api.inspector(A, 2, kind=9)


def test_schedule_round_trips(built_lib):
    a = synth.laplacian((30, 30))
    A = api.CSRMatrix(900, 900, *a)
    s = api.inspector(A, 4, kind=api.INSPECT_VT_GEMM, tile_m=40000, b_cols=16, c_cols=16)
    t = api.FusedSchedule.deserialize(s.serialize())
    assert common.same_schedule(s, t) and np.array_equal(s.stats, t.stats)
    u = api.FusedSchedule.from_arrays(s.n1, s.ptr1, s.ptr2, s.id, s.type, s.ker_begin)
    assert common.same_schedule(s, u)
    with pytest.raises(api.TileFusionError):
        api.FusedSchedule.deserialize(s.serialize()[:20])
    with pytest.raises(api.TileFusionError):
        api.FusedSchedule.from_arrays(2, [0, 1, 2], [0, 5, 3], np.zeros(3), np.zeros(3))


def test_library_exports_every_declared_symbol(built_lib):
    """Every function include/tile_fusion_b200.h declares is exported by the shared library."""
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "include", "tile_fusion_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(tf_[a-z0-9_]+)\s*\(", text))
    assert len(declared) >= 30
    lib = C.CDLL(built_lib)
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    assert b"sm_100a" in lib_version(lib)


def lib_version(lib):
    lib.tf_version.restype = C.c_char_p
    return lib.tf_version()


def test_product_does_not_touch_the_oracle():
    """The package must not import, load or name anything under oracle/."""
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dirpath, _, files in os.walk(os.path.join(root, "tile_fusion_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), os.path.join(dirpath, f)


def test_executors_fail_loudly_without_a_gpu(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    a = synth.laplacian((8, 8))
    A = api.CSRMatrix(64, 64, *a)
    with pytest.raises(api.TileFusionError) as e:
        api.Plan("spmm_spmm", A, n_cols=32)
    assert e.value.code == _lib.TF_ERR_CUDA


def test_fingerprint_sees_refilled_arrays():
    """The README-level executors cache their plan per matrix; the key must change when the arrays are refilled
    in place or when another matrix takes an old object's place."""
    a = synth.laplacian((6, 5, 4))
    A = api.CSRMatrix(len(a[0]) - 1, len(a[0]) - 1, *a)
    f0 = A.fingerprint()
    assert f0 == A.fingerprint()
    A.Ax *= 2.0
    assert A.fingerprint() != f0
    b = synth.laplacian((6, 5, 4))
    assert api.CSRMatrix(len(b[0]) - 1, len(b[0]) - 1, *b).fingerprint()[:5] == f0[:5]   # same matrix, other arrays
