"""One rank of the multi-GPU parity check (launched by tests/test_gpu_multi.py through torch.distributed.run).

Every rank owns a row block of a 3-D Laplacian, runs the partitioned chains with the halo exchange over NCCL
and compares its rows of D with an fp64 product of the whole chain computed on the host."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

from tests import common  # noqa: E402
from tile_fusion_b200 import distributed, partition, synth  # noqa: E402


def main():
    import scipy.sparse as sp
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    for dims, n, k in (((24, 20, 10 * world), 128, 64), ((40, 33 * world), 32, 16), ((16, 12, 6 * world), 100, 36)):
        n_rows = int(np.prod(dims))
        full = synth.laplacian(dims)
        A64 = sp.csr_matrix((full[2].astype(np.float64), full[1], full[0]), shape=(n_rows, n_rows))
        bounds = partition.row_bounds(None, n_rows, world)
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        a_rows = synth.laplacian_rows(dims, r0, r1)
        mine = partition.halo_of(a_rows[1], r0, r1)
        halos = [None] * world
        dist.all_gather_object(halos, mine)
        lay = partition.make_layout(rank, bounds, halos)
        # SpMM-SpMM
        c = synth.uniform(3, (n_rows, n)) - 0.5
        ids, fi = partition.compact_columns(a_rows[1])
        rc = distributed.RankChain("spmm_spmm", lay, a_rows, n, first_rows=(a_rows[0], fi, a_rows[2], len(ids)), device=dev)
        c_ext = torch.from_numpy(np.ascontiguousarray(c[ids])).to(dev)
        d = torch.full((r1 - r0, n), float("nan"), device=dev)
        for _ in range(2):
            rc.step(c_ext, None, d, dist=dist)
            rc.plan.status()
            want = (A64 @ (A64 @ c.astype(np.float64)))[r0:r1]
            common.assert_close(d.cpu().numpy(), want, f"rank {rank} SpMM-SpMM {dims}")
        # GeMM-SpMM
        b, w = synth.uniform(2, (n_rows, k)) - 0.5, synth.uniform(4, (k, n)) - 0.5
        rg = distributed.RankChain("gemm_spmm", lay, a_rows, n, k=k, device=dev)
        bd, wd = torch.from_numpy(np.ascontiguousarray(b[r0:r1])).to(dev), torch.from_numpy(w).to(dev)
        d.fill_(float("nan"))
        rg.step(bd, wd, d, dist=dist)
        rg.plan.status()
        want = (A64 @ (b.astype(np.float64) @ w.astype(np.float64)))[r0:r1]
        common.assert_close(d.cpu().numpy(), want, f"rank {rank} GeMM-SpMM {dims}")
        # the same two chains through the library's own multi-GPU entry points (partition in C++, ncclSend / ncclRecv)
        nat = distributed.NativeRankChain("spmm_spmm", rank, world, r0, r1, a_rows, n, dist=dist, device=dev)
        assert (nat.info["c_first"], nat.info["c_rows"]) == (int(ids[0]), len(ids)), nat.info
        assert nat.info["halo_rows"] == len(lay.halo_ids) and nat.info["boundary_rows"] == len(lay.boundary_rows)
        d2 = torch.full((r1 - r0, n), float("nan"), device=dev)
        for _ in range(2):
            nat.step(c_ext, None, d2)
        nat.status()
        want = (A64 @ (A64 @ c.astype(np.float64)))[r0:r1]
        common.assert_close(d2.cpu().numpy(), want, f"rank {rank} native SpMM-SpMM {dims}")
        # a traced step: every phase is recorded and ends inside the step
        nat.trace(True)
        nat.step(c_ext, None, d2)
        tr = nat.trace(False)
        assert tr is not None and all(0 <= tr[k] <= tr["step_done"] + 0.02 for k in tr), tr   # (two streams: 0.02 ms of slack)
        common.assert_close(d2.cpu().numpy(), want, f"rank {rank} native SpMM-SpMM {dims}, traced step")
        nat.close()
        # the same with the halo rows sent through ncclSend / ncclRecv instead of the copy engines: same bits
        nat = distributed.NativeRankChain("spmm_spmm", rank, world, r0, r1, a_rows, n, dist=dist, device=dev, exchange=-1)
        d3 = torch.full((r1 - r0, n), float("nan"), device=dev)
        nat.step(c_ext, None, d3)
        nat.status()
        assert torch.equal(d3, d2), "the two exchange paths differ"
        nat.close()
        nat = distributed.NativeRankChain("gemm_spmm", rank, world, r0, r1, a_rows, n, k=k, dist=dist, device=dev)
        d2.fill_(float("nan"))
        nat.step(bd, wd, d2)
        nat.status()
        assert torch.equal(d2, d), "native GeMM-SpMM differs from the torch.distributed rank program"
        nat.close()
        dist.barrier()
    if rank == 0:
        print("multi-GPU parity ok on", world, "ranks")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
