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


class NativeRankChain:
    """The same rank program behind one C call per step (tf_multi_*): the partition arrays are derived in the
    library (the halo lists are all-gathered over NCCL), the exchange is ncclSend / ncclRecv on the plan's own
    stream.  `dist` (torch.distributed, any backend) only carries the 128-byte NCCL id from rank 0 to the others."""

    def __init__(self, chain, rank, world, r0, r1, a_rows, n_cols, *, k=0, dist=None, device=None, **plan_kw):
        import ctypes as C

        import torch

        from . import _lib
        L = _lib.lib()
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_char * 128)()
            _lib.check(L.tf_comm_unique_id(buf))
            ident = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
        if world > 1:
            t = ident.to(self.device) if dist.get_backend() == "nccl" else ident
            dist.broadcast(t, 0)
            ident = t.cpu()
        raw = bytes(ident.numpy().tobytes())
        self._comm = C.c_void_p()
        _lib.check(L.tf_comm_create(raw, world, rank, C.byref(self._comm)))
        ap, ai, ax = a_rows
        ap = np.ascontiguousarray(ap, dtype=np.int32)
        ai = np.ascontiguousarray(ai, dtype=np.int64)
        ax = np.ascontiguousarray(ax, dtype=np.float32)
        o = _lib.PlanOpts(plan_kw.get("mode", 0), plan_kw.get("rows_per_block", 0), 0, -1, 0, 0, 0, None, 0, 0, 0, 0, 0, 0,
                          plan_kw.get("exchange", 0))
        self._h = C.c_void_p()
        _lib.check(L.tf_multi_plan(self._comm, 0 if chain == "spmm_spmm" else 1, int(r0), int(r1), ap.ctypes.data,
                                   ai.ctypes.data, ax.ctypes.data, int(k), int(n_cols), C.byref(o), C.byref(self._h)))
        info = (C.c_longlong * 8)()
        _lib.check(L.tf_multi_info(self._h, info))
        keys = ["rows", "halo_rows", "boundary_rows", "c_first", "c_rows", "send_peers", "recv_peers", "threads"]
        self.info = dict(zip(keys, [int(x) for x in info]))

    def step(self, in0, in1, out, w_transposed=False, relu=False, stream=None):
        from . import _lib
        from .api import _stream_ptr
        _lib.check(_lib.lib().tf_multi_exec(self._h, in0.data_ptr(), in1.data_ptr() if in1 is not None else None,
                                            int(w_transposed), int(relu), out.data_ptr(),
                                            stream if stream is not None else _stream_ptr()))

    def status(self, stream=None):
        from . import _lib
        from .api import _stream_ptr
        _lib.check(_lib.lib().tf_multi_status(self._h, stream if stream is not None else _stream_ptr()))

    def trace(self, on=True):
        """Switches step tracing on / off and returns the last traced step's times (ms from its start) as a dict,
        or None when no traced step has run."""
        import ctypes
        from . import _lib
        ms = (ctypes.c_float * 5)()
        _lib.check(_lib.lib().tf_multi_trace(self._h, int(bool(on)), ms))
        if ms[4] < 0:
            return None
        return dict(zip(("phase0_done", "exchange_done", "phase2_done", "phase1_done", "step_done"), (float(v) for v in ms)))

    def close(self):
        from . import _lib
        if getattr(self, "_h", None):
            _lib.lib().tf_multi_free(self._h)
            self._h = None
        if getattr(self, "_comm", None):
            _lib.lib().tf_comm_free(self._comm)
            self._comm = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def native_layout(rank, bounds, halos):
    """The partition arrays of `rank` as the library derives them (tf_partition_layout): (boundary_rows, recv, send)
    with recv / send as lists of (peer, start, count, contiguous)."""
    import ctypes as C

    from . import _lib
    world = len(bounds) - 1
    b = np.ascontiguousarray(bounds, dtype=np.int64)
    hp = np.zeros(world + 1, np.int64)
    np.cumsum([len(h) for h in halos], out=hp[1:])
    hid = np.ascontiguousarray(np.concatenate([np.asarray(h, dtype=np.int64) for h in halos]) if hp[-1] else np.zeros(1, np.int64))
    br, rv, sd = C.c_void_p(), C.c_void_p(), C.c_void_p()
    nb, nr, ns = C.c_longlong(), C.c_int(), C.c_int()
    _lib.check(_lib.lib().tf_partition_layout(int(rank), world, b.ctypes.data, hp.ctypes.data, hid.ctypes.data, C.byref(br),
                                              C.byref(nb), C.byref(rv), C.byref(nr), C.byref(sd), C.byref(ns)))

    def take(p, n):
        a = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_longlong)), shape=(max(n, 1),)).copy()[:n]
        _lib.lib().tf_free(p)
        return a
    return (take(br, nb.value), [tuple(int(v) for v in q) for q in take(rv, 4 * nr.value).reshape(-1, 4)],
            [tuple(int(v) for v in q) for q in take(sd, 4 * ns.value).reshape(-1, 4)])
