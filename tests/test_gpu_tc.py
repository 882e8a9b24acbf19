"""The tcgen05 3xTF32 dense producer against an fp64 product (tolerance of tests/common.py)."""
import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import _lib, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n,wt", [(300, 64, 64, False), (1000, 100, 256, False), (4096, 256, 256, True),
                                      (129, 36, 48, False), (128, 32, 16, True), (70000, 64, 64, False)])
def test_tc_gemm_matches_fp64(built_lib, m, k, n, wt):
    import torch
    L = _lib.lib()
    b = synth.uniform(2, (m, k))
    w = synth.uniform(3, (k, n))
    want = b.astype(np.float64) @ w.astype(np.float64)
    bd = torch.from_numpy(b).cuda()
    wd = torch.from_numpy(np.ascontiguousarray(w.T) if wt else w).cuda()
    t = torch.full((m, n), float("nan"), device="cuda")
    _lib.check(L.tf_gemm_tc_dev(bd.data_ptr(), wd.data_ptr(), int(wt), m, k, n, t.data_ptr(),
                                torch.cuda.current_stream().cuda_stream))
    rel, mx = common.assert_close(t.cpu().numpy(), want, f"tc gemm {m}x{k}x{n}")
    assert rel < 2e-6, rel  # 3xTF32 keeps fp32-level accuracy


def test_tc_gemm_rejects_unsupported_shapes(built_lib):
    import torch
    L = _lib.lib()
    x = torch.zeros(64 * 64, device="cuda")
    for k, n in ((30, 64), (64, 47), (64, 512)):
        rc = L.tf_gemm_tc_dev(x.data_ptr(), x.data_ptr(), 0, 8, k, n, x.data_ptr(), None)
        assert rc == _lib.TF_ERR_UNSUPPORTED


def test_tensor_core_plan_refuses_unaligned_output(built_lib):
    """A GeMM-SpMM plan with the tensor-core producer on a graph (no gather tiles) stores D with 16-byte
    vectors: an output that starts off a 16-byte boundary is refused before anything is launched."""
    import torch
    from tile_fusion_b200 import api
    a = synth.rmat_gcn(7, 3000, 14)
    A = api.CSRMatrix(3000, 3000, *a)
    plan = api.Plan("gemm_spmm", A, k=64, n_cols=64)
    b = torch.zeros((3000, 64), device="cuda")
    w = torch.zeros((64, 64), device="cuda")
    d = torch.full((3000 * 64 + 1,), 7.0, device="cuda")
    with pytest.raises(_lib.TileFusionError) as e:
        plan.gemm_spmm(b, w, d[1:].view(3000, 64))
    assert e.value.code == _lib.TF_ERR_ARG
    torch.cuda.synchronize()
    assert bool((d == 7.0).all())          # nothing ran
    plan.gemm_spmm(b, w, d[:3000 * 64].view(3000, 64))
    plan.status()
    plan.close()
