"""Parity at the full sizes of the benchmark configurations, through properties that do not need the CPU
oracle to run the whole job: single columns against an fp64 product, exact integer results for a constant
operand, linearity, and bit-identity between the executor's modes.
Tolerance: rel-L2 <= 1e-5 and max-abs <= 1e-4 * ||D||_inf (tests/common.py)."""
import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import _lib, api, synth

pytestmark = pytest.mark.gpu


def _scipy_csr(t, n):
    import scipy.sparse as sp
    return sp.csr_matrix((t[2].astype(np.float64), t[1], t[0]), shape=(n, n))


def _fill(torch, t, seed):
    _lib.check(_lib.lib().tf_fill_uniform(t.data_ptr(), t.numel(), seed, 0, torch.cuda.current_stream().cuda_stream))


def test_spmm_spmm_128cubed(built_lib):
    """SpMM-SpMM on the 128^3 7-point Laplacian, N = 128 (2 097 152 rows, 14.6 M nonzeros)."""
    import torch
    dims, n_cols = (128, 128, 128), 128
    n = int(np.prod(dims))
    t = synth.laplacian(dims)
    A = api.CSRMatrix(n, n, *t)
    S = _scipy_csr(t, n)
    plans = {"march": api.Plan("spmm_spmm", A, n_cols=n_cols),
             "pipeline": api.Plan("spmm_spmm", A, n_cols=n_cols, lattice_march=-1),
             "two_cta_tiles": api.Plan("spmm_spmm", A, n_cols=n_cols, tile_pipeline=-1, lattice_march=-1),
             "unfused_direct": api.Plan("spmm_spmm", A, n_cols=n_cols, mode=api.MODE_UNFUSED, tile_slots=-1)}
    assert plans["march"].info()["threads"] == 128      # the plane-marching kernel: the intermediate stays on chip
    assert plans["pipeline"].info()["threads"] == 672
    c = torch.empty((n, n_cols), device="cuda")
    _fill(torch, c, 3)
    out = {}
    for name, p in plans.items():
        d = torch.full((n, n_cols), float("nan"), device="cuda")
        p.spmm_spmm(c, d)
        p.status()
        out[name] = d
    # every mode adds the same products in the same order
    assert torch.equal(out["march"], out["unfused_direct"])
    assert torch.equal(out["pipeline"], out["unfused_direct"])
    assert torch.equal(out["two_cta_tiles"], out["unfused_direct"])
    # single columns against fp64
    d = out["march"]
    for j in (0, 77, 127):
        cj = c[:, j].double().cpu().numpy()
        common.assert_close(d[:, j].cpu().numpy(), S @ (S @ cj), f"column {j}")
    # constant operand: every product and sum is a small integer, so the result is exact
    c.fill_(1.0)
    plans["march"].spmm_spmm(c, d)
    plans["march"].status()
    want = S @ (S @ np.ones(n))
    assert np.array_equal(d[:, 5].cpu().numpy().astype(np.float64), want)
    assert torch.equal(d, d[:, :1].expand(-1, n_cols))
    # linearity: chain(x + 2 y) = chain(x) + 2 chain(y)
    x, y = torch.empty_like(c), torch.empty_like(c)
    _fill(torch, x, 11)
    _fill(torch, y, 12)
    dx, dy, dz = torch.empty_like(c), torch.empty_like(c), torch.empty_like(c)
    p = plans["march"]
    p.spmm_spmm(x, dx)
    p.spmm_spmm(y, dy)
    p.spmm_spmm(x + 2 * y, dz)
    p.status()
    common.assert_close(dz.cpu().numpy(), (dx.double() + 2 * dy.double()).cpu().numpy(), "linearity")
    for p in plans.values():
        p.close()


def test_gemm_spmm_256squared(built_lib, oracle):
    """GeMM-SpMM on the 256^2 5-point Laplacian, K = N = 64: small enough for the CPU oracle as a whole."""
    import torch
    dims, k, n_cols = (256, 256), 64, 64
    n = int(np.prod(dims))
    t = synth.laplacian(dims)
    A = api.CSRMatrix(n, n, *t)
    b, w = synth.uniform(2, (n, k)), synth.uniform(3, (k, n_cols))
    want, _ = oracle.gemm_spmm(t, b, w, oracle.inspect_fixed(t[0], t[1], 4, 2048))
    for kw in (dict(), dict(tensor_cores=-1), dict(mode=api.MODE_UNFUSED)):
        plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols, **kw)
        d = torch.full((n, n_cols), float("nan"), device="cuda")
        plan.gemm_spmm(torch.from_numpy(b).cuda(), torch.from_numpy(w).cuda(), d)
        plan.status()
        common.assert_close(d.cpu().numpy(), want, f"GeMM-SpMM 256^2 {kw}")
        plan.close()


def test_gemm_spmm_large_slab(built_lib):
    """GeMM-SpMM with K = N = 256 on a 256 x 256 x 32 slab of the 256^3 case (2 097 152 rows): columns of D
    against an fp64 product formed with torch and scipy."""
    import torch
    dims, k, n_cols = (256, 256, 32), 256, 256
    n = int(np.prod(dims))
    t = synth.laplacian(dims)
    A = api.CSRMatrix(n, n, *t)
    S = _scipy_csr(t, n)
    b, w = torch.empty((n, k), device="cuda"), torch.empty((k, n_cols), device="cuda")
    _fill(torch, b, 2)
    _fill(torch, w, 3)
    outs = []
    for kw in (dict(), dict(mode=api.MODE_UNFUSED)):
        plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols, **kw)
        d = torch.full((n, n_cols), float("nan"), device="cuda")
        plan.gemm_spmm(b, w, d)
        plan.status()
        outs.append(d)
        plan.close()
    assert torch.equal(outs[0], outs[1])
    for j in (0, 131, 255):
        tj = (b.double() @ w[:, j].double()).cpu().numpy()
        common.assert_close(outs[0][:, j].cpu().numpy(), S @ tj, f"column {j}")
