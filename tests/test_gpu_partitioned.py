"""The row-block partitioned chains, every rank emulated in turn on one GPU: phase 0 of all ranks,
the halo exchange as plain device copies, then phases 1 and 2.  No launch waits for another."""
import numpy as np
import pytest

from tests import common
from tile_fusion_b200 import api, distributed, partition, synth

pytestmark = pytest.mark.gpu


def _exchange_by_copy(ranks):
    for r in ranks:
        for seg in r.lay.recv:
            src = ranks[seg.peer]
            s = next(x for x in src.lay.send if x.peer == r.lay.rank)
            rows = src.sendbuf[s.start:s.start + s.count] if s.index is None else \
                src.sendbuf.index_select(0, src._gather_idx[r.lay.rank])
            r.halobuf[seg.start:seg.start + seg.count].copy_(rows)


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("spec,by", [(("lap", (12, 10, 9)), "rows"), (("rmat_gcn", 5, 1500, 8), "nnz")])
def test_partitioned_gemm_spmm(built_lib, oracle, world, spec, by):
    import torch
    a = common.matrix(spec)
    n, k, nc = len(a[0]) - 1, 40, 64
    b, w = synth.uniform(2, (n, k)), synth.uniform(3, (k, nc))
    want, _ = oracle.gemm_spmm(a, b, w, oracle.inspect_fixed(a[0], a[1], 2, 64))
    bounds = partition.row_bounds(a[0], n, world, by)
    rows = [(a[0][bounds[g]:bounds[g + 1] + 1] - a[0][bounds[g]], a[1][a[0][bounds[g]]:a[0][bounds[g + 1]]].astype(np.int64),
             a[2][a[0][bounds[g]]:a[0][bounds[g + 1]]]) for g in range(world)]
    halos = [partition.halo_of(rows[g][1], int(bounds[g]), int(bounds[g + 1])) for g in range(world)]
    ranks = [distributed.RankChain("gemm_spmm", partition.make_layout(g, bounds, halos), rows[g], nc, k=k,
                                   rows_per_block=16) for g in range(world)]
    wd = torch.from_numpy(w).cuda()
    bd = [torch.from_numpy(b[bounds[g]:bounds[g + 1]]).cuda() for g in range(world)]
    out = [torch.full((int(bounds[g + 1] - bounds[g]), nc), float("nan"), device="cuda") for g in range(world)]
    for g, r in enumerate(ranks):
        if len(r.lay.boundary_rows):
            r.plan.phase(0, bd[g], wd, None)
    _exchange_by_copy(ranks)
    for g, r in enumerate(ranks):
        r.plan.phase(1, bd[g], wd, out[g])
        r.plan.phase(2, bd[g], wd, out[g])
        r.plan.status()
    got = torch.cat(out).cpu().numpy()
    common.assert_close(got, want, f"partitioned GeMM-SpMM world={world}")


@pytest.mark.parametrize("world,dims,nc,march", [(2, (10, 8, 16), 32, True), (4, (10, 8, 16), 32, True),
                                                  (3, (34, 18, 9), 48, True), (2, (9, 8, 16), 32, False)])
def test_partitioned_spmm_spmm(built_lib, oracle, world, dims, nc, march):
    """march: the ranks' slabs run on the plane-marching kernel (phase 1: the planes that need no plane of the
    intermediate from a neighbour; phase 2: the first / last plane, with the received planes)."""
    import torch
    a = synth.laplacian(dims)
    n = len(a[0]) - 1
    c = synth.uniform(3, (n, nc))
    want, _ = oracle.spmm_spmm(a, a, c, oracle.inspect_fixed(a[0], a[1], 2, 64))
    bounds = partition.row_bounds(None, n, world)
    ranks, cd, out = [], [], []
    rows = [synth.laplacian_rows(dims, int(bounds[g]), int(bounds[g + 1])) for g in range(world)]
    halos = [partition.halo_of(rows[g][1], int(bounds[g]), int(bounds[g + 1])) for g in range(world)]
    for g in range(world):
        ids, fi = partition.compact_columns(rows[g][1])
        lay = partition.make_layout(g, bounds, halos)
        ranks.append(distributed.RankChain("spmm_spmm", lay, rows[g], nc, rows_per_block=16,
                                           first_rows=(rows[g][0], fi, rows[g][2], len(ids))))
        assert (ranks[-1].plan.info()["threads"] == 128) == march, ranks[-1].plan.info()
        cd.append(torch.from_numpy(c[ids]).cuda())  # own rows of C plus ghost rows
        out.append(torch.full((lay.m, nc), float("nan"), device="cuda"))
    for g, r in enumerate(ranks):
        r.plan.phase(0, cd[g], None, None)
    _exchange_by_copy(ranks)
    for g, r in enumerate(ranks):
        r.plan.phase(1, cd[g], None, out[g])
        r.plan.phase(2, cd[g], None, out[g])
        r.plan.status()
    common.assert_close(torch.cat(out).cpu().numpy(), want, f"partitioned SpMM-SpMM world={world}")
