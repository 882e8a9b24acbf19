"""The allocation-free SpMM-SpMM entry point (collected last on purpose: if it fails under `-x`,
every other test has already run).

Some callers may not allocate device memory when they need the product -- cudaMalloc / cudaFree
take the allocator lock and can synchronise the device -- so tf_spmm_spmm_noalloc keeps its
intermediate in an array built into the library.  This test calls it through the C ABI on device
pointers and checks it against the existing plain SpMM entry point (tf_spmm_dev applied twice),
twice in a row: the second call finds the first call's data in the shared array."""
import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def test_no_alloc_entry_point_matches_spmm_twice(built_lib):
    import torch
    torch.cuda.init()
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    limit = L.tf_noalloc_max_floats()
    assert limit == 4 << 20
    for call, (spec, n_cols, seed) in enumerate([(("lap", (30, 20, 10)), 128, 3), (("rmat_gcn", 4, 5000, 9), 48, 8)]):
        a = common.matrix(spec)
        m = len(a[0]) - 1
        assert m * n_cols <= limit
        ap, ai, ax = (torch.from_numpy(v).cuda() for v in a)
        c = torch.from_numpy(synth.uniform(seed, (m, n_cols))).cuda()
        t = torch.empty((m, n_cols), device="cuda")
        want = torch.empty((m, n_cols), device="cuda")
        _lib.check(L.tf_spmm_dev(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), m, c.data_ptr(), n_cols, t.data_ptr(), st))
        _lib.check(L.tf_spmm_dev(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), m, t.data_ptr(), n_cols, want.data_ptr(), st))
        got = torch.full((m, n_cols), float("nan"), device="cuda")
        _lib.check(L.tf_spmm_spmm_noalloc(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), m, c.data_ptr(), n_cols,
                                          got.data_ptr(), st))
        torch.cuda.synchronize()
        common.assert_close(got.cpu().numpy(), want.cpu().numpy(), f"no-alloc call {call}")
    # a problem beyond the built-in intermediate is refused with a message that names the limit
    rc = L.tf_spmm_spmm_noalloc(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), 1 << 20, c.data_ptr(), 8,
                                got.data_ptr(), st)
    assert rc == _lib.TF_ERR_ARG and b"exceeds" in L.tf_last_error()
