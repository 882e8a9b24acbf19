"""Host logic of the row-block partition, and the halo exchange choreography over gloo (2 ranks)."""
import os
import socket

import numpy as np
import pytest

from tile_fusion_b200 import distributed, partition, synth


def test_bounds_and_layouts_are_consistent():
    dims = (6, 5, 8)
    n = 240
    full = synth.laplacian(dims)
    for world in (1, 2, 3, 4):
        bounds = partition.row_bounds(None, n, world)
        assert bounds[0] == 0 and bounds[-1] == n and (np.diff(bounds) >= n // world).all()
        rows = [synth.laplacian_rows(dims, int(bounds[g]), int(bounds[g + 1])) for g in range(world)]
        assert np.array_equal(np.concatenate([r[1] for r in rows]), full[1])
        assert np.array_equal(np.concatenate([r[2] for r in rows]), full[2])
        halos = [partition.halo_of(rows[g][1], int(bounds[g]), int(bounds[g + 1])) for g in range(world)]
        lays = [partition.make_layout(g, bounds, halos) for g in range(world)]
        for g, lay in enumerate(lays):
            assert sum(s.count for s in lay.recv) == len(lay.halo_ids)
            for s in lay.recv:  # what g receives from p is what p sends to g, in the same order
                t = next(x for x in lays[s.peer].send if x.peer == g)
                assert t.count == s.count
                sent_local = lays[s.peer].boundary_rows[t.start:t.start + t.count] if t.index is None \
                    else lays[s.peer].boundary_rows[t.index]
                np.testing.assert_array_equal(sent_local + bounds[s.peer], lay.halo_ids[s.start:s.start + s.count])
            loc = partition.localize_columns(rows[g][1], lay)
            assert loc.min() >= 0 and loc.max() < lay.m + len(lay.halo_ids)
            hid = np.concatenate([lay.halo_ids, [-1]])  # world 1: no halo
            back = np.where(loc < lay.m, loc + lay.r0, hid[np.clip(loc - lay.m, 0, len(hid) - 1)])
            np.testing.assert_array_equal(back, rows[g][1])


@pytest.mark.parametrize("spec,world,by", [(("lap", (6, 5, 8)), 3, "rows"), (("lap", (40, 33)), 4, "rows"),
                                           (("rmat_gcn", 5, 1500, 8), 3, "nnz"), (("rmat_gcn", 9, 700, 6), 2, "rows")])
def test_native_partition_matches(built_lib, spec, world, by):
    """tf_partition_layout (the C++ partition the multi-GPU entry points use) against partition.make_layout: boundary
    rows, receive and send segments -- graphs give send segments that are not contiguous in the send buffer."""
    from tests import common
    a = common.matrix(spec)
    n = len(a[0]) - 1
    bounds = partition.row_bounds(a[0], n, world, by)
    halos = []
    for g in range(world):
        p0, p1 = a[0][bounds[g]], a[0][bounds[g + 1]]
        halos.append(partition.halo_of(a[1][p0:p1].astype(np.int64), int(bounds[g]), int(bounds[g + 1])))
    for g in range(world):
        lay = partition.make_layout(g, bounds, halos)
        br, rv, sd = distributed.native_layout(g, bounds, halos)
        assert np.array_equal(br, lay.boundary_rows)
        assert rv == [(s.peer, s.start, s.count, 1) for s in lay.recv]
        assert sd == [(s.peer, s.start, s.count, int(s.index is None)) for s in lay.send]


def test_nnz_balanced_bounds():
    ap, ai, ax = synth.rmat_gcn(3, 4000, 10)
    b = partition.row_bounds(ap, 4000, 4, by="nnz")
    per = np.diff(ap[b])
    assert per.sum() == ap[-1] and per.max() < 1.5 * per.mean()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, dims, nc, ret):
    import torch
    import torch.distributed as dist
    import scipy.sparse as sp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = int(np.prod(dims))
        bounds = partition.row_bounds(None, n, world)
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        ap, ai, ax = synth.laplacian_rows(dims, r0, r1)
        mine = partition.halo_of(ai, r0, r1)
        halos = [None] * world
        dist.all_gather_object(halos, mine)
        lay = partition.make_layout(rank, bounds, halos)
        # the library's own (C++) partition gives the same arrays from the gathered halo lists
        br, rv, sd = distributed.native_layout(rank, bounds, halos)
        assert np.array_equal(br, lay.boundary_rows)
        assert rv == [(s.peer, s.start, s.count, 1) for s in lay.recv]
        assert sd == [(s.peer, s.start, s.count, int(s.index is None)) for s in lay.send]
        # numpy stands in for the device kernels: T rows of this rank = B_local @ W
        b = synth.uniform(2, (n, 8))[r0:r1].astype(np.float64)
        w = synth.uniform(3, (8, nc)).astype(np.float64)
        t_local = b @ w
        send = torch.from_numpy(t_local[lay.boundary_rows])            # phase 0
        halo = torch.zeros((len(lay.halo_ids), nc), dtype=torch.float64)
        ops = [dist.P2POp(dist.isend, send[s.start:s.start + s.count].contiguous(), s.peer) for s in lay.send]
        ops += [dist.P2POp(dist.irecv, halo[s.start:s.start + s.count], s.peer) for s in lay.recv]
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        t_all = np.concatenate([t_local, halo.numpy()])               # local rows, then halo rows
        a_loc = sp.csr_matrix((ax.astype(np.float64), partition.localize_columns(ai, lay), ap),
                              shape=(lay.m, lay.m + len(lay.halo_ids)))
        ret[rank] = (r0, a_loc @ t_all)
    finally:
        dist.destroy_process_group()


def test_halo_exchange_two_ranks_gloo():
    import torch.multiprocessing as mp
    import scipy.sparse as sp
    dims, nc, world = (5, 4, 6), 3, 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, dims, nc, ret), nprocs=world, join=True)
    a = synth.laplacian(dims)
    n = int(np.prod(dims))
    A = sp.csr_matrix((a[2].astype(np.float64), a[1], a[0]), shape=(n, n))
    want = A @ (synth.uniform(2, (n, 8)).astype(np.float64) @ synth.uniform(3, (8, nc)).astype(np.float64))
    got = np.concatenate([ret[g][1] for g in range(world)])
    np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-12)


def test_multi_entry_points_reject_bad_arguments(built_lib):
    """The multi-GPU entry points answer with a status, not a crash, when handed nothing (no GPU, no NCCL needed)."""
    import ctypes as C

    from tile_fusion_b200 import _lib
    L = _lib.lib()
    ms = (C.c_float * 5)()
    assert L.tf_multi_trace(None, 1, ms) == _lib.TF_ERR_ARG
    assert L.tf_multi_status(None, None) == _lib.TF_ERR_ARG
    assert L.tf_multi_exec(None, None, None, 0, 0, None, None) == _lib.TF_ERR_ARG
    out = C.c_void_p()
    assert L.tf_comm_create(None, 2, 0, C.byref(out)) == _lib.TF_ERR_ARG
    assert L.tf_comm_from_nccl(None, 2, 0, C.byref(out)) == _lib.TF_ERR_ARG
    assert L.tf_multi_plan(None, 0, 0, 10, None, None, None, 0, 8, None, C.byref(out)) == _lib.TF_ERR_ARG
    assert b"null" in L.tf_last_error() or b"bad" in L.tf_last_error()
