"""The allocation-free SpMM-SpMM entry point (collected last on purpose: if it fails under `-x`,
every other test has already run).

Some callers may not allocate device memory when they need the product -- cudaMalloc / cudaFree
take the allocator lock and can synchronise the device -- so tf_spmm_spmm_noalloc keeps its
intermediate in an array built into the library.  This test calls it through the C ABI on device
pointers and checks it against the existing plain SpMM entry point (tf_spmm_dev applied twice) and
against the CPU oracle's two CSR products, several calls in a row: every call after the first finds the
previous call's data in the shared array.  The cases cover the 16-byte vector path, the 8-byte one, the
scalar one (odd width) and operands that start one float off a 16-byte boundary."""
import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def test_no_alloc_entry_point_matches_spmm_twice(built_lib, oracle):
    import torch
    torch.cuda.init()
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    limit = L.tf_noalloc_max_floats()
    assert limit == 4 << 20
    cases = [(("lap", (30, 20, 10)), 128, 3, 0), (("rmat_gcn", 4, 5000, 9), 48, 8, 0), (("lap", (40, 33)), 47, 5, 0),
             (("rmat_gcn", 6, 3000, 7), 64, 9, 1)]
    for call, (spec, n_cols, seed, shift) in enumerate(cases):
        a = common.matrix(spec)
        m = len(a[0]) - 1
        assert m * n_cols <= limit
        ap, ai, ax = (torch.from_numpy(v).cuda() for v in a)
        ch = synth.uniform(seed, (m, n_cols))
        # shift = 1: C and D are views that begin one float after a 16-byte boundary
        c = torch.empty(m * n_cols + shift, device="cuda")[shift:].view(m, n_cols)
        c.copy_(torch.from_numpy(ch))
        t = torch.empty((m, n_cols), device="cuda")
        want = torch.empty((m, n_cols), device="cuda")
        _lib.check(L.tf_spmm_dev(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), m, c.data_ptr(), n_cols, t.data_ptr(), st))
        _lib.check(L.tf_spmm_dev(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), m, t.data_ptr(), n_cols, want.data_ptr(), st))
        got = torch.full((m * n_cols + shift,), float("nan"), device="cuda")[shift:].view(m, n_cols)
        _lib.check(L.tf_spmm_spmm_noalloc(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), m, c.data_ptr(), n_cols,
                                          got.data_ptr(), st))
        torch.cuda.synchronize()
        common.assert_close(got.cpu().numpy(), want.cpu().numpy(), f"no-alloc call {call} against tf_spmm_dev twice")
        cpu = oracle.spmm(a[0], a[1], a[2], oracle.spmm(a[0], a[1], a[2], ch))
        common.assert_close(got.cpu().numpy(), cpu, f"no-alloc call {call} against the oracle")
    # a problem beyond the built-in intermediate is refused with a message that names the limit
    rc = L.tf_spmm_spmm_noalloc(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), 1 << 20, c.data_ptr(), 8,
                                got.data_ptr(), st)
    assert rc == _lib.TF_ERR_ARG and b"exceeds" in L.tf_last_error()
