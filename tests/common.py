"""Shared helpers of the test-suite: golden fixtures and tolerance checks."""
import json
import os

import numpy as np

from tile_fusion_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# north-star tolerance against the reference CPU executor
REL_L2 = 1e-5
MAX_ABS_REL = 1e-4


def manifest():
    with open(os.path.join(GOLDEN, "manifest.json")) as f:
        return json.load(f)


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def matrix(spec):
    if spec[0] == "lap":
        return synth.laplacian(tuple(spec[1]))
    if spec[0] == "rmat_gcn":
        return synth.rmat_gcn(spec[1], spec[2], spec[3])
    raise ValueError(spec)


def assert_close(got, want, what=""):
    """rel-L2 <= 1e-5 and max-abs <= 1e-4 * ||want||_inf."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), what + ": non-finite output"
    den = np.linalg.norm(want)
    rel = np.linalg.norm(got - want) / (den if den > 0 else 1.0)
    mx = np.abs(got - want).max() if got.size else 0.0
    lim = MAX_ABS_REL * (np.abs(want).max() if want.size else 1.0)
    assert rel <= REL_L2, f"{what}: rel-L2 {rel:.3e} > {REL_L2}"
    assert mx <= lim + 1e-30, f"{what}: max-abs {mx:.3e} > {lim:.3e}"
    return rel, mx


def same_schedule(a, b):
    """a, b: objects with n1, ptr1, ptr2, id, type, ker_begin."""
    if a.n1 != b.n1:
        return False
    for x, y in ((a.ptr1, b.ptr1), (a.ptr2, b.ptr2), (a.id, b.id), (a.type, b.type)):
        if len(x) != len(y) or not np.array_equal(x, y):
            return False
    if (a.ker_begin is None) != (b.ker_begin is None):
        return False
    return a.ker_begin is None or np.array_equal(a.ker_begin, b.ker_begin)


def assert_sums(d, g, what=""):
    """Whole-output sums of a fixture that keeps only some rows: sum and sum of squares of D."""
    d64 = np.asarray(d, dtype=np.float64)
    scale = np.sqrt(float(g["sq"]) * d64.size)
    assert abs(d64.sum() - float(g["total"])) <= 1e-5 * scale, what + ": sum of D"
    assert abs((d64 ** 2).sum() - float(g["sq"])) <= 1e-5 * float(g["sq"]), what + ": sum of squares of D"
