"""One rank of a row-block partitioned chain: three launches around one halo exchange.

    phase 0   produce the boundary rows of T into the send buffer          (main stream)
    exchange  NCCL send/recv of those rows into the neighbours' halo rows   (comm stream)
    phase 1   every producer block and every consumer block that reads no halo row (main stream,
              overlaps the exchange)
    phase 2   the consumer blocks that read halo rows, after the receive    (main stream)

No kernel waits for another launch: the ordering is by stream events only.
"""
from __future__ import annotations

import numpy as np

from . import api, partition


class _DevView:
    """A device buffer owned by the library, presented through __cuda_array_interface__."""

    def __init__(self, ptr: int, rows: int, cols: int):
        self.__cuda_array_interface__ = {"shape": (rows, cols), "typestr": "<f4", "data": (ptr, False),
                                         "version": 3, "strides": None}


def _as_tensor(ptr, rows, cols, device):
    import torch
    if rows == 0:
        return torch.empty((0, cols), device=device, dtype=torch.float32)
    return torch.as_tensor(_DevView(ptr, rows, cols), device=device)


class RankChain:
    """chain = "gemm_spmm" (first operand dense m x k) or "spmm_spmm" (first operator = rows of B
    with columns already compacted to the rank's rows of C, see partition.compact_columns)."""

    def __init__(self, chain, lay: partition.RankLayout, a_rows, n_cols, *, k=0, first_rows=None, device=None,
                 **plan_kw):
        import torch
        self.lay, self.chain, self.n_cols = lay, chain, n_cols
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        ap, ai_g, ax = a_rows
        A = api.CSRMatrix(lay.m, lay.m + len(lay.halo_ids), ap, partition.localize_columns(ai_g, lay), ax)
        kw = dict(halo_rows=len(lay.halo_ids), boundary_rows=lay.boundary_rows.astype(np.int32), **plan_kw)
        if chain == "gemm_spmm":
            self.plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols, **kw)
        else:
            fp, fi, fx, n_c_rows = first_rows
            B = api.CSRMatrix(lay.m, n_c_rows, fp, fi, fx)
            self.plan = api.Plan("spmm_spmm", A, B=B, n_cols=n_cols, **kw)
        sp, sr, hp, hr = self.plan.exchange_buffers()
        self.sendbuf = _as_tensor(sp, sr, n_cols, self.device)
        self.halobuf = _as_tensor(hp, hr, n_cols, self.device)
        self.comm_stream = torch.cuda.Stream(device=self.device)
        self._ready, self._arrived = torch.cuda.Event(), torch.cuda.Event()
        self._ops = None
        self._gather_idx = {s.peer: torch.as_tensor(s.index, device=self.device) for s in lay.send
                            if s.index is not None}

    def exchange_ops(self, dist):
        """P2P ops of one halo exchange (send buffer segments out, halo segments in).  The op objects
        name fixed device buffers, so they are built once and reused by every step."""
        if self._ops is not None:
            return self._ops
        ops, gathers = [], []
        for s in self.lay.send:
            if s.index is None:
                t = self.sendbuf[s.start:s.start + s.count]
            else:  # non-contiguous rows: gathered into a staging tensor before each send
                t = self.sendbuf.new_empty((s.count, self.n_cols))
                gathers.append((t, self._gather_idx[s.peer]))
            ops.append(dist.P2POp(dist.isend, t, s.peer))
        for s in self.lay.recv:
            ops.append(dist.P2POp(dist.irecv, self.halobuf[s.start:s.start + s.count], s.peer))
        self._ops = (ops, gathers)
        return self._ops

    def step(self, in0, in1, out, dist=None, w_transposed=False, relu=False, exchange=None):
        """One pass.  `dist` = torch.distributed (NCCL) or None with `exchange(self)` a callable that
        fills the halo buffer some other way (single-process tests)."""
        import torch
        main = torch.cuda.current_stream(self.device)
        has_x = len(self.lay.send) + len(self.lay.recv) > 0
        if len(self.lay.boundary_rows):
            self.plan.phase(0, in0, in1, None, w_transposed, relu)
        if has_x and dist is not None:
            self._ready.record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self._ready)
                ops, gathers = self.exchange_ops(dist)
                for t, idx in gathers:
                    torch.index_select(self.sendbuf, 0, idx, out=t)
                for r in dist.batch_isend_irecv(ops):
                    r.wait()
                self._arrived.record(self.comm_stream)
            self.plan.phase(1, in0, in1, out, w_transposed, relu)
            main.wait_event(self._arrived)
        else:
            self.plan.phase(1, in0, in1, out, w_transposed, relu)
            if exchange is not None:
                exchange(self)
        self.plan.phase(2, in0, in1, out, w_transposed, relu)
