"""Parity of the CUDA executors (through the C ABI) with the CPU oracle and the golden vectors.
Tolerance: rel-L2 <= 1e-5 and max-abs <= 1e-4 * ||D||_inf (tests/common.py)."""
import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import api, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda(built_lib):
    import torch
    torch.cuda.init()
    return torch


def _csr(t):
    n = len(t[0]) - 1
    return api.CSRMatrix(n, n, *t)


def _dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _sched(A, kind, n_cols, k=0, threads=4):
    if kind == 1:
        return api.inspector(A, threads, kind=1, iter_per_partition=max(8, A.M // 37))
    if kind == 2:
        return api.inspector(A, threads, kind=2, tile_m=40 * 4 * n_cols * 3, b_cols=n_cols)
    return api.inspector(A, threads, kind=3, tile_m=4 * (k * n_cols + 120 * (k + n_cols)), b_cols=k, c_cols=n_cols)


MATS = {
    "lap2d_40x33": ("lap", (40, 33)),
    "lap3d_14": ("lap", (14, 14, 14)),
    "lap1d_3000": ("lap", (3000,)),
    "rmat_3000": ("rmat_gcn", 7, 3000, 14),
}


@pytest.mark.parametrize("n_cols", [128, 64, 47, 100, 256, 8, 300])
def test_spmm_kernel(torch_cuda, oracle, n_cols):
    torch = torch_cuda
    from tile_fusion_b200 import _lib
    a = common.matrix(MATS["rmat_3000"])
    x = synth.uniform(5, (3000, n_cols))
    want = oracle.spmm(a[0], a[1], a[2], x)
    out = torch.empty((3000, n_cols), device="cuda")
    ap, ai, ax, xd = (_dev(torch, v) for v in (a[0], a[1], a[2], x))
    _lib.check(_lib.lib().tf_spmm_dev(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), 3000, xd.data_ptr(), n_cols,
                                      out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    common.assert_close(out.cpu().numpy(), want, f"spmm N={n_cols}")


@pytest.mark.parametrize("mat", list(MATS))
@pytest.mark.parametrize("n_cols", [128, 32, 47, 64, 100])
def test_spmm_spmm_all_modes(torch_cuda, oracle, mat, n_cols):
    torch = torch_cuda
    a = common.matrix(MATS[mat])
    A = _csr(a)
    c = synth.uniform(3, (A.M, n_cols))
    want, _ = oracle.spmm_spmm(a, a, c, oracle.inspect_fixed(a[0], a[1], 2, 64))
    cd = _dev(torch, c)
    results = {}
    variants = [("stream_ring", dict(mode=api.MODE_STREAM, rows_per_block=16, slack_blocks=4, ring_bytes=1 << 30,
                                     tile_slots=-1)),
                ("stream_default", dict(mode=api.MODE_STREAM)),
                ("stream_tile_pipeline", dict(mode=api.MODE_STREAM, lattice_march=-1)),
                ("stream_two_cta_tiles", dict(mode=api.MODE_STREAM, tile_pipeline=-1, lattice_march=-1)),
                ("stream_noring", dict(mode=api.MODE_STREAM, ring_bytes=-1, rows_per_block=8, tile_slots=-1)),
                ("tiled_ring", dict(mode=api.MODE_STREAM, tile_slots=160, tile_max_bz=2, ring_bytes=1 << 30,
                                    slack_blocks=3)),
                ("tiled_unfused", dict(mode=api.MODE_UNFUSED, tile_slots=400)),
                ("unfused", dict(mode=api.MODE_UNFUSED, tile_slots=-1)),
                ("sched_fixed", dict(mode=api.MODE_SCHEDULE, schedule=_sched(A, 1, n_cols))),
                ("sched_vt", dict(mode=api.MODE_SCHEDULE, schedule=_sched(A, 2, n_cols)))]
    for name, kw in variants:
        plan = api.Plan("spmm_spmm", A, n_cols=n_cols, **kw)
        d = torch.full((A.M, n_cols), float("nan"), device="cuda")
        for _ in range(2):  # twice: the executor state must rewind
            plan.spmm_spmm(cd, d)
        plan.status()
        results[name] = d.cpu().numpy()
        common.assert_close(results[name], want, f"{mat} N={n_cols} {name}")
        if name == "stream_default" and mat == "lap3d_14" and n_cols % 4 == 0:
            assert plan.info()["threads"] == 128, plan.info()  # star stencil on a 3-D grid: the plane-marching kernel
        if name == "stream_tile_pipeline" and mat.startswith("lap") and n_cols % 4 == 0:
            assert plan.info()["threads"] == 672, plan.info()  # both operators tiled: the tile pipeline runs it
        if name == "stream_two_cta_tiles" and mat.startswith("lap") and n_cols % 4 == 0:
            assert plan.info()["threads"] == 512, plan.info()
        if name == "stream_ring" and mat.startswith("lap"):
            assert 0 < plan.info()["ring_rows"] < A.M
        if name == "tiled_unfused" and mat.startswith("lap") and n_cols % 4 == 0:
            assert plan.tile_info()["consumer"][3] > 0, plan.tile_info()
        if name == "tiled_ring" and mat.startswith("lap"):
            assert 0 < plan.info()["ring_rows"] < A.M, plan.info()
        plan.close()
    # every mode adds the same products in the same order (rows heavy enough to be split over a
    # CTA in stream mode are reduced in another order, so the graph case is left out)
    if mat.startswith("lap"):
        for name in results:
            np.testing.assert_array_equal(results[name], results["unfused"], err_msg=name)


@pytest.mark.parametrize("dims,n_cols", [((40, 34, 9), 100), ((18, 16, 5), 128), ((16, 8, 3), 4), ((34, 20, 20), 48)])
def test_plane_march_shapes(torch_cuda, oracle, dims, n_cols):
    """The plane-marching kernel on grids that are no multiples of its 16 x 8 tiles, widths that are no multiples
    of its 16-column chunks, and two different operators: against the oracle's two CSR products, and bit for
    bit against the unfused CSR executor."""
    torch = torch_cuda
    a = synth.laplacian(dims)
    n = len(a[0]) - 1
    rows = np.repeat(np.arange(n), np.diff(a[0]))
    bx = (a[2] * (1.0 + (rows % 2)) * np.where(a[1] > rows, 0.5, 1.0)).astype(np.float32)
    b = (a[0], a[1], bx)
    c = synth.uniform(3, (n, n_cols))
    cd = _dev(torch, c)
    for first, what in ((a, "B = A"), (b, "B != A")):
        A, B = _csr(a), _csr(first)
        want = oracle.spmm(a[0], a[1], a[2], oracle.spmm(first[0], first[1], first[2], c))
        plan = api.Plan("spmm_spmm", A, B=None if first is a else B, n_cols=n_cols)
        assert plan.info()["threads"] == 128, plan.info()
        d = torch.full((n, n_cols), float("nan"), device="cuda")
        for _ in range(2):
            plan.spmm_spmm(cd, d)
        plan.status()
        common.assert_close(d.cpu().numpy(), want, f"plane march {dims} N={n_cols} {what}")
        ref_plan = api.Plan("spmm_spmm", A, B=None if first is a else B, n_cols=n_cols, mode=api.MODE_UNFUSED, tile_slots=-1,
                            lattice_march=-1)
        d0 = torch.empty_like(d)
        ref_plan.spmm_spmm(cd, d0)
        ref_plan.status()
        assert torch.equal(d, d0), what
        # the host-pointer call of the same plan (grids of 8 planes or more: one launch per slab of planes between
        # the copy streams) must give the same bits
        dh = np.full((n, n_cols), np.nan, np.float32)
        plan.spmm_spmm_host(c, dh)
        assert np.array_equal(dh, d.cpu().numpy()), what + " (host pointers)"
        plan.close()
        ref_plan.close()


@pytest.mark.parametrize("dims,k,n_cols", [((18, 16, 9), 40, 64), ((34, 20, 6), 64, 112)])
def test_gemm_spmm_marching_consumer(torch_cuda, oracle, dims, k, n_cols):
    """GeMM-SpMM on a 3-D grid operator: the tensor-core producer's rows are consumed by the plane-marching kernel
    (identity as first operator).  Against the oracle, and bit for bit against the ticket executor's consumer."""
    torch = torch_cuda
    a = synth.laplacian(dims)
    n = len(a[0]) - 1
    A = _csr(a)
    b, w = synth.uniform(2, (n, k)), synth.uniform(3, (k, n_cols))
    want, _ = oracle.gemm_spmm(a, b, w, oracle.inspect_fixed(a[0], a[1], 2, 64))
    bd, wd = _dev(torch, b), _dev(torch, w)
    got = {}
    for name, lm in (("march", 0), ("ticket", -1)):
        plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols, lattice_march=lm)
        assert (plan.info()["threads"] == 128) == (name == "march"), plan.info()
        d = torch.full((n, n_cols), float("nan"), device="cuda")
        for _ in range(2):
            plan.gemm_spmm(bd, wd, d)
        plan.status()
        got[name] = d.cpu().numpy()
        common.assert_close(got[name], want, f"GeMM-SpMM {name} consumer {dims}")
        plan.close()
    np.testing.assert_array_equal(got["march"], got["ticket"])


def _nine_point(nx, ny):
    import scipy.sparse as sp
    x, y = np.meshgrid(np.arange(nx), np.arange(ny))
    r = (y * nx + x).ravel()
    rows, cols, vals = [], [], []
    for dy in (-1, 0, 1):
        for dx in (-1, 0, 1):
            ok = ((x + dx >= 0) & (x + dx < nx) & (y + dy >= 0) & (y + dy < ny)).ravel()
            rows.append(r[ok]); cols.append((r + dy * nx + dx)[ok])
            vals.append(np.full(ok.sum(), 8.0 if dx == 0 and dy == 0 else -1.0, np.float32))
    S = sp.csr_matrix((np.concatenate(vals), (np.concatenate(rows), np.concatenate(cols))), shape=(nx * ny, nx * ny))
    S.sort_indices()
    return S.indptr.astype(np.int32), S.indices.astype(np.int32), S.data.astype(np.float32)


def _perturbed_band(n, per_row, half_width, seed):
    import scipy.sparse as sp
    rng = np.random.default_rng(seed)
    rows = np.repeat(np.arange(n), per_row)
    cols = np.clip(rows + rng.integers(-half_width, half_width + 1, size=rows.size), 0, n - 1)
    S = sp.csr_matrix((rng.uniform(-1, 1, rows.size).astype(np.float32), (rows, cols)), shape=(n, n))
    S.sum_duplicates()
    S.sort_indices()
    return S.indptr.astype(np.int32), S.indices.astype(np.int32), S.data.astype(np.float32)


@pytest.mark.parametrize("which", ["nine_point", "band", "rcm_graph"])
def test_generic_gather_tiles(torch_cuda, oracle, which):
    """Patterns that are no 5- / 7-point lattices get gather tiles from runs of consecutive rows (the 9-point
    operator, a randomly perturbed band, a graph after the RCM ordering): tiles exist, and the tiled executors agree
    with the oracle's two CSR products and, bit for bit, with the untiled executor."""
    torch = torch_cuda
    if which == "nine_point":
        a = _nine_point(60, 50)
    elif which == "band":
        a = _perturbed_band(4000, 12, 40, 1)
    else:
        g = synth.rmat_gcn(7, 3000, 14)
        G = api.CSRMatrix(3000, 3000, *g)
        P = api.permute(G, api.rcm_order(G))
        a = (P.Ap, P.Ai, P.Ax)
    A = _csr(a)
    for n_cols in (64, 100):
        c = synth.uniform(3, (A.M, n_cols))
        want = oracle.spmm(a[0], a[1], a[2], oracle.spmm(a[0], a[1], a[2], c))
        cd = _dev(torch, c)
        outs = {}
        for name, kw in (("pipeline", dict()), ("two_cta", dict(tile_pipeline=-1)), ("untiled", dict(tile_slots=-1))):
            plan = api.Plan("spmm_spmm", A, n_cols=n_cols, **kw)
            if name != "untiled" and n_cols % 4 == 0:
                assert plan.tile_info()["consumer"][3] > 0, (which, name, plan.tile_info())
            d = torch.full((A.M, n_cols), float("nan"), device="cuda")
            plan.spmm_spmm(cd, d)
            plan.status()
            outs[name] = d
            common.assert_close(d.cpu().numpy(), want, f"{which} N={n_cols} {name}")
            plan.close()
        if which != "rcm_graph":  # (a graph's rows of 256 nonzeros or more are reduced by a whole CTA when untiled: another order)
            assert torch.equal(outs["pipeline"], outs["untiled"]) and torch.equal(outs["two_cta"], outs["untiled"])
    # the dense-producer chain on the same tiles
    k, n_cols = 32, 64
    b, w = synth.uniform(2, (A.M, k)), synth.uniform(4, (k, n_cols))
    plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols)
    assert plan.tile_info()["consumer"][3] > 0
    d = torch.full((A.M, n_cols), float("nan"), device="cuda")
    plan.gemm_spmm(_dev(torch, b), _dev(torch, w), d)
    plan.status()
    t = (b.astype(np.float64) @ w.astype(np.float64)).astype(np.float32)
    common.assert_close(d.cpu().numpy(), oracle.spmm(a[0], a[1], a[2], t), f"{which} GeMM-SpMM")
    plan.close()


def test_spmm_spmm_two_operators_and_host_path(torch_cuda, oracle):
    a = common.matrix(MATS["lap2d_40x33"])
    b = common.matrix(("rmat_gcn", 3, 40 * 33, 5))
    A, B = _csr(a), _csr(b)
    c = synth.uniform(3, (A.M, 64))
    want, _ = oracle.spmm_spmm(a, b, c, oracle.inspect_fixed(a[0], a[1], 2, 64))
    d = np.zeros((A.M, 64), np.float32)
    api.spMMSpMMExecutor(A, B, api.Matrix(A.M, 64, c), api.Matrix(A.M, 64, d), None, 8)
    common.assert_close(d, want, "host path, A != B")
    s = api.inspector(A, 4, kind=2, tile_m=60000, b_cols=64)
    d2 = np.zeros_like(d)
    api.spMMSpMMExecutor(A, A, api.Matrix(A.M, 64, c), api.Matrix(A.M, 64, d2), s, 8, mode=api.MODE_SCHEDULE)
    want2, _ = oracle.spmm_spmm(a, a, c, oracle.inspect_variable(2, a[0], a[1], 4, 60000, 64))
    common.assert_close(d2, want2, "host path, schedule mode")


@pytest.mark.parametrize("mat", ["lap2d_40x33", "rmat_3000"])
@pytest.mark.parametrize("k,n_cols", [(64, 64), (100, 256), (256, 47), (17, 33)])
def test_gemm_spmm_all_modes(torch_cuda, oracle, mat, k, n_cols):
    torch = torch_cuda
    a = common.matrix(MATS[mat])
    A = _csr(a)
    b = synth.uniform(2, (A.M, k))
    w = synth.uniform(3, (k, n_cols))
    so = oracle.inspect_fixed(a[0], a[1], 2, 64)
    want, _ = oracle.gemm_spmm(a, b, w, so)
    bd, wd, wtd = _dev(torch, b), _dev(torch, w), _dev(torch, w.T)
    for name, kw in [("stream", dict(mode=api.MODE_STREAM)),
                     ("stream_small", dict(mode=api.MODE_STREAM, rows_per_block=16, slack_blocks=3)),
                     ("unfused", dict(mode=api.MODE_UNFUSED)),
                     ("sched_fixed", dict(mode=api.MODE_SCHEDULE, schedule=_sched(A, 1, n_cols))),
                     ("sched_vt", dict(mode=api.MODE_SCHEDULE, schedule=_sched(A, 3, n_cols, k)))]:
        plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols, **kw)
        d = torch.full((A.M, n_cols), float("nan"), device="cuda")
        plan.gemm_spmm(bd, wd, d)
        plan.status()
        common.assert_close(d.cpu().numpy(), want, f"{mat} {k}x{n_cols} {name}")
        d.fill_(float("nan"))
        plan.gemm_spmm(bd, wtd, d, w_transposed=True, relu=True)
        plan.status()
        common.assert_close(d.cpu().numpy(), np.maximum(want, 0), f"{mat} {k}x{n_cols} {name} transposed+relu")
        plan.close()


def test_gemm_spmm_host_executor(torch_cuda, oracle):
    a = common.matrix(MATS["lap3d_14"])
    A = _csr(a)
    b, w = synth.uniform(2, (A.M, 48)), synth.uniform(3, (48, 96))
    want, _ = oracle.gemm_spmm(a, b, w, oracle.inspect_fixed(a[0], a[1], 2, 64))
    d = np.zeros((A.M, 96), np.float32)
    api.geMMSpMMExecutor(A, api.Matrix(A.M, 48, b), api.Matrix(48, 96, w), api.Matrix(A.M, 96, d), None, 4)
    common.assert_close(d, want, "geMMSpMMExecutor host")


@pytest.mark.parametrize("kq,nv", [(64, 128), (32, 64), (100, 47), (160, 256)])
def test_sddmm_spmm(torch_cuda, oracle, kq, nv):
    torch = torch_cuda
    a = synth.rmat_pattern(4, 2500, 20)
    A = api.CSRMatrix(2500, 2500, *a)
    q, k, v = synth.normal(2, (2500, kq), 0.125), synth.normal(3, (2500, kq), 0.125), synth.normal(4, (2500, nv), 0.125)
    want = oracle.sddmm_spmm(a, q, k, v)
    d = torch.full((2500, nv), float("nan"), device="cuda")
    api.sddmmSpMMExecutor(A, api.Matrix(2500, kq, _dev(torch, q)), api.Matrix(2500, kq, _dev(torch, k)),
                          api.Matrix(2500, nv, _dev(torch, v)), api.Matrix(2500, nv, d))
    torch.cuda.synchronize()
    common.assert_close(d.cpu().numpy(), want, f"SDDMM-SpMM {kq}/{nv}")
    dh = np.zeros((2500, nv), np.float32)
    api.sddmmSpMMExecutor(A, api.Matrix(2500, kq, q), api.Matrix(2500, kq, k), api.Matrix(2500, nv, v),
                          api.Matrix(2500, nv, dh))
    np.testing.assert_array_equal(dh, d.cpu().numpy())


@pytest.mark.parametrize("name", [k for k, v in common.manifest().items() if "kq" in v])
def test_sddmm_spmm_against_reference_sampled_values(torch_cuda, oracle, name):
    """D = S V with S the values the reference's sddmm_cpu produced (tests/golden), multiplied by the pinned CSR
    SpMM of the oracle: the CUDA chain never stores S, so it is checked through D."""
    torch = torch_cuda
    case = common.manifest()[name]
    spec, kq, nv = case["matrix"], case["kq"], 64
    a = synth.rmat_pattern(spec[1], spec[2], spec[3])
    n = len(a[0]) - 1
    q, k, v = synth.normal(2, (n, kq), 0.125), synth.normal(3, (n, kq), 0.125), synth.normal(4, (n, nv), 0.125)
    want = oracle.spmm(a[0], a[1], common.golden(name)["S"], v)
    d = torch.full((n, nv), float("nan"), device="cuda")
    api.sddmmSpMMExecutor(api.CSRMatrix(n, n, *a), api.Matrix(n, kq, _dev(torch, q)), api.Matrix(n, kq, _dev(torch, k)),
                          api.Matrix(n, nv, _dev(torch, v)), api.Matrix(n, nv, d))
    torch.cuda.synchronize()
    common.assert_close(d.cpu().numpy(), want, name)


def test_gcn_two_layers(torch_cuda, oracle):
    torch = torch_cuda
    g = synth.rmat_gcn(6, 4000, 25)
    A = api.CSRMatrix(4000, 4000, *g)
    x, w1, w2 = synth.normal(2, (4000, 100)), synth.glorot(3, 256, 100), synth.glorot(4, 47, 256)
    out, plans = api.gcn_forward(A, _dev(torch, x), _dev(torch, w1), _dev(torch, w2))
    torch.cuda.synchronize()
    common.assert_close(out.cpu().numpy(), oracle.gcn2(g, x, w1, w2), "2-layer GCN")


@pytest.mark.parametrize("name", [k for k, v in common.manifest().items() if "chain" in v])
def test_golden_outputs(torch_cuda, name):
    """Outputs of the unmodified reference on seeded inputs (tests/golden)."""
    torch = torch_cuda
    case = common.manifest()[name]
    a = common.matrix(case["matrix"])
    A = _csr(a)
    prm = case["params"]
    s = api.inspector(A, prm["threads"], kind=case["kind"], iter_per_partition=prm.get("iter_per_part", 1),
                      tile_m=prm.get("tile_m", 1), b_cols=prm.get("bcol", 1), c_cols=prm.get("ccol", 1))
    g = common.golden(name)
    want = g["D"]
    rows = g["rows"] if "rows" in g else np.arange(A.M)   # the larger fixtures keep every 4th row and two sums
    for mode in (api.MODE_STREAM, api.MODE_SCHEDULE):
        d = np.zeros((A.M, want.shape[1]), np.float32)
        if case["chain"] == "spmm_spmm":
            c = synth.uniform(3, (A.M, case["dims"]["n"]))
            api.spMMSpMMExecutor(A, A, api.Matrix(*c.shape, c), api.Matrix(*d.shape, d), s, 2, mode=mode)
        else:
            b = synth.uniform(2, (A.M, case["dims"]["k"]))
            w = synth.uniform(3, (case["dims"]["k"], case["dims"]["n"]))
            api.geMMSpMMExecutor(A, api.Matrix(*b.shape, b), api.Matrix(*w.shape, w), api.Matrix(*d.shape, d), s, 2,
                                 mode=mode)
        common.assert_close(d[rows], want, f"{name} mode {mode}")
        if "total" in g:
            common.assert_sums(d, g, f"{name} mode {mode}")


def test_device_fills_match_host_generators(torch_cuda):
    torch = torch_cuda
    from tile_fusion_b200 import _lib
    n = 100003
    t = torch.empty(n, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib().tf_fill_uniform(t.data_ptr(), n, 3, 1000, st))
    np.testing.assert_array_equal(t.cpu().numpy(), synth.uniform(3, (n,), start=1000))
    _lib.check(_lib.lib().tf_fill_normal(t.data_ptr(), n, 4, 77, 0.125, st))
    np.testing.assert_allclose(t.cpu().numpy(), synth.normal(4, (n,), 0.125, start=77), rtol=2e-5, atol=1e-6)


def test_edge_shapes(torch_cuda, oracle):
    torch = torch_cuda
    # one row, one column; empty rows; N = 1
    ap = np.array([0, 1], np.int32)
    A = api.CSRMatrix(1, 1, ap, np.array([0], np.int32), np.array([2.0], np.float32))
    d = np.zeros((1, 1), np.float32)
    api.spMMSpMMExecutor(A, A, api.Matrix(1, 1, np.array([[3.0]], np.float32)), api.Matrix(1, 1, d), None)
    assert d[0, 0] == 12.0
    n = 257
    rows = [np.array([], np.int32) if r % 5 == 0 else np.array(sorted({r, (r * 7) % n, n - 1 - r}), np.int32)
            for r in range(n)]
    ap = np.zeros(n + 1, np.int32)
    ap[1:] = np.cumsum([len(r) for r in rows])
    ai = np.concatenate(rows).astype(np.int32)
    ax = synth.uniform(9, (len(ai),))
    t = (ap, ai, ax)
    A = api.CSRMatrix(n, n, *t)
    c = synth.uniform(3, (n, 5))
    want = oracle.spmm(ap, ai, ax, oracle.spmm(ap, ai, ax, c))
    d = np.full((n, 5), np.nan, np.float32)
    api.spMMSpMMExecutor(A, A, api.Matrix(n, 5, c), api.Matrix(n, 5, d), None)
    common.assert_close(d, want, "empty rows")
    with pytest.raises(ValueError):
        api.spMMSpMMExecutor(A, A, api.Matrix(n, 5, c), api.Matrix(n, 4, np.zeros((n, 4), np.float32)), None)
    with pytest.raises(api.TileFusionError):
        api.Plan("gemm_spmm", A, k=0, n_cols=4)


def test_heavy_row_split_over_cta(torch_cuda, oracle):
    """A row far above the per-block nonzero cap is reduced by the whole CTA."""
    torch = torch_cuda
    n = 4096
    rows = [np.arange(n, dtype=np.int32) if r in (5, 4000) else np.array([r], np.int32) for r in range(n)]
    ap = np.zeros(n + 1, np.int32)
    ap[1:] = np.cumsum([len(r) for r in rows])
    ai = np.concatenate(rows)
    ax = synth.uniform(8, (len(ai),))
    A = api.CSRMatrix(n, n, ap, ai, ax)
    c = synth.uniform(3, (n, 128))
    want = oracle.spmm(ap, ai, ax, oracle.spmm(ap, ai, ax, c))
    d = np.zeros((n, 128), np.float32)
    api.spMMSpMMExecutor(A, A, api.Matrix(n, 128, c), api.Matrix(n, 128, d), None)
    common.assert_close(d, want, "heavy rows")


def _hub(n, hubs, seed):
    rows = [np.arange(hubs[r], dtype=np.int32) if r in hubs else np.unique(np.array([r, (r * 7 + 1) % n], np.int32))
            for r in range(n)]
    ap = np.zeros(n + 1, np.int32)
    ap[1:] = np.cumsum([len(r) for r in rows])
    ai = np.concatenate(rows)
    return ap, ai, (synth.uniform(seed, (len(ai),)) - 0.5).astype(np.float32)


@pytest.mark.parametrize("n_cols", [128, 47])
def test_rows_cut_into_segments(torch_cuda, oracle, n_cols):
    """Rows above the segment size are shared by several CTAs, which add their parts atomically into
    rows zeroed before the pass; the order of the adds varies, the tolerance covers it."""
    torch = torch_cuda
    n = 12000
    a = _hub(n, {5: 11000, 7000: 9000, 11999: 4097, 300: 700}, 8)
    A = api.CSRMatrix(n, n, *a)
    c = synth.uniform(3, (n, n_cols)) - 0.5
    want = oracle.spmm(*a, oracle.spmm(*a, c))
    for mode in (api.MODE_STREAM, api.MODE_UNFUSED):
        plan = api.Plan("spmm_spmm", A, n_cols=n_cols, mode=mode)
        d = torch.full((n, n_cols), float("nan"), device="cuda")
        cd = _dev(torch, c)
        for _ in range(2):  # the second call must start from zeroed rows again
            plan.spmm_spmm(cd, d)
            plan.status()
            common.assert_close(d.cpu().numpy(), want, f"segments SpMM-SpMM mode {mode}")
        plan.close()
    dh = np.zeros((n, n_cols), np.float32)
    api.spMMSpMMExecutor(A, A, api.Matrix(n, n_cols, c), api.Matrix(n, n_cols, dh), None)
    common.assert_close(dh, want, "segments SpMM-SpMM host")
    # dense producer, ReLU applied after the atomic adds
    k = 64
    b, w = synth.uniform(2, (n, k)) - 0.5, synth.uniform(4, (k, n_cols)) - 0.5
    want_g = np.maximum(oracle.spmm(*a, (b.astype(np.float64) @ w.astype(np.float64)).astype(np.float32)), 0)
    plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols)
    d = torch.full((n, n_cols), float("nan"), device="cuda")
    plan.gemm_spmm(_dev(torch, b), _dev(torch, w), d, relu=True)
    plan.status()
    common.assert_close(d.cpu().numpy(), want_g, "segments GeMM-SpMM + ReLU")
    plan.close()
    # SDDMM-SpMM
    q, kk, v = synth.normal(2, (n, 32), 0.125), synth.normal(3, (n, 32), 0.125), synth.normal(4, (n, n_cols), 0.125)
    want_s = oracle.sddmm_spmm(a, q, kk, v)
    d = torch.full((n, n_cols), float("nan"), device="cuda")
    api.sddmmSpMMExecutor(A, api.Matrix(n, 32, _dev(torch, q)), api.Matrix(n, 32, _dev(torch, kk)),
                          api.Matrix(n, n_cols, _dev(torch, v)), api.Matrix(n, n_cols, d))
    torch.cuda.synchronize()
    common.assert_close(d.cpu().numpy(), want_s, "segments SDDMM-SpMM")


def test_bounded_wait_reports_timeout(torch_cuda):
    """Failure detection without a GPU fault: consumers of a halo plan are launched without the
    producers they wait for; the wait runs out, the kernel returns and the host reads the status."""
    torch = torch_cuda
    a = synth.laplacian((8, 8, 4))
    m, halo = 256, 0
    # a plan with a (fake) halo: columns of the last rows point to 4 extra rows
    ap, ai, ax = a
    ai2 = ai.copy()
    ai2[-3:] = [m, m + 1, m + 3]
    A = api.CSRMatrix(m, m + 4, ap, ai2, ax)
    plan = api.Plan("spmm_spmm", A, B=api.CSRMatrix(m, m, *a), n_cols=32, halo_rows=4,
                    boundary_rows=np.array([0, 1], np.int32))
    plan.set_wait_limit(200)
    c = torch.zeros((m, 32), device="cuda")
    d = torch.zeros((m, 32), device="cuda")
    plan.phase(2, c, None, d)  # phase 1 never ran: nothing publishes the producer blocks
    with pytest.raises(api.TileFusionError) as e:
        plan.status()
    assert e.value.code == -4
    # the plan stays usable
    plan.set_wait_limit(1 << 22)
    plan.phase(0, c, None, None)
    plan.phase(1, c, None, d)
    plan.phase(2, c, None, d)
    plan.status()
    assert float(d.abs().sum()) == 0.0
