"""Host-side mirror of the reference's operator interface, over the C ABI.

The reference documents (README.md:21-38)::

    FusedSchedule inspector(CSRMatrix A, int NumThreads)
    spMMSpMMExecutor(CSRMatrix A, CSRMatrix B, Matrix C, Matrix D, FusedSchedule schedule, int NumThreads)
    geMMSpMMExecutor(CSRMatrix A, Matrix  B, Matrix C, Matrix D, FusedSchedule schedule, int NumThreads)
    CSRMatrix(int M, int N, int* Ap, int* Ai, float* Ax);  Matrix(int M, int N, float* Data)

with D = A * B * C.  The same names and argument meaning are kept here.  Dense
operands may be numpy arrays (host path: copied to the device and back inside the
call) or CUDA torch tensors (device path: no copies, runs on torch's current
stream).  Everything executes in the CUDA library; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import (INSPECT_FIXED, INSPECT_VT_GEMM, INSPECT_VT_SPMM, INSPECT_VT_SPMM_THREADS, MODE_SCHEDULE,
                   MODE_STREAM, MODE_UNFUSED, TileFusionError, check)

__all__ = ["CSRMatrix", "Matrix", "FusedSchedule", "ScheduleParameters", "inspector", "spMMSpMMExecutor",
           "geMMSpMMExecutor", "sddmmSpMMExecutor", "Plan", "gcn_forward", "TileFusionError"]


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class CSRMatrix:
    """CSRMatrix(M, N, Ap, Ai, Ax) -- README.md:37.  Host arrays, int32 / fp32, not copied if already so."""

    def __init__(self, M, N, Ap, Ai, Ax):
        self.M, self.N = int(M), int(N)
        self.Ap, self.Ai, self.Ax = _i32(Ap), _i32(Ai), _f32(Ax)
        if self.Ap.shape[0] != self.M + 1:
            raise ValueError("CSRMatrix: Ap must have M + 1 entries")
        if self.Ai.shape[0] != self.Ap[-1] or self.Ax.shape[0] != self.Ap[-1]:
            raise ValueError("CSRMatrix: Ai and Ax must have Ap[M] entries")

    @property
    def nnz(self):
        return int(self.Ap[-1])

    def _c(self) -> _lib.Csr:
        return _lib.Csr(self.M, self.N, self.Ap.ctypes.data, self.Ai.ctypes.data, self.Ax.ctypes.data)

    def fingerprint(self):
        """Sampled checksum (size, up to 2048 evenly spaced column ids and values).  The plan cache of the
        README-level executors keys on it beside the object, so that an object id reused by another matrix, or
        arrays refilled in place, get a new plan.  A change that touches none of the sampled entries is not seen:
        make a new CSRMatrix for new values."""
        nnz = self.nnz
        step = max(1, nnz // 2048)
        return (self.M, self.N, nnz, int(self.Ai[::step].astype(np.int64).sum()),
                self.Ax[::step].tobytes().__hash__(), self.Ap.ctypes.data, self.Ai.ctypes.data, self.Ax.ctypes.data)


class Matrix:
    """Matrix(M, N, Data) -- README.md:38.  Data: numpy array (host) or CUDA torch tensor (device)."""

    def __init__(self, M, N, Data):
        self.M, self.N = int(M), int(N)
        if isinstance(Data, np.ndarray):
            if Data.dtype != np.float32 or not Data.flags["C_CONTIGUOUS"]:
                raise ValueError("Matrix: host data must be a C-contiguous float32 array")
            self.on_device = False
        else:  # torch tensor
            if not (Data.is_cuda and Data.is_contiguous() and Data.dtype.is_floating_point and Data.element_size() == 4):
                raise ValueError("Matrix: device data must be a contiguous float32 CUDA tensor")
            self.on_device = True
        if int(np.prod(Data.shape)) != self.M * self.N:
            raise ValueError("Matrix: Data must hold M*N values")
        self.Data = Data

    @property
    def ptr(self) -> int:
        return self.Data.data_ptr() if self.on_device else self.Data.ctypes.data


@dataclass
class ScheduleParameters:
    """sym_lib::ScheduleParameters (fusion/include/sparse-fusion/Fusion_Defs.h:21-55) plus the dense widths
    the variable-tile inspectors take.  The defaults are the reference sweep's mid point
    (fusion/scripts/run_exp.sh mode 7)."""
    kind: int = INSPECT_FIXED
    num_threads: int = 8
    iter_per_partition: int = 2048
    tile_m: int = 1_250_000
    b_cols: int = 32
    c_cols: int = 32
    data_size: int = 4


class FusedSchedule:
    """The reference-format schedule (sym_lib::MultiDimensionalSet): n1 levels, ptr1, ptr2, id, type, ker_begin."""

    def __init__(self, handle: int, params: ScheduleParameters | None = None):
        self._h = C.c_void_p(handle)
        self.params = params
        L = _lib.lib()
        n1, npart, nid, hk = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        check(L.tf_schedule_dims(self._h, C.byref(n1), C.byref(npart), C.byref(nid), C.byref(hk)))
        ptrs = [C.c_void_p() for _ in range(5)]
        check(L.tf_schedule_arrays(self._h, *[C.byref(p) for p in ptrs]))

        def view(p, n):
            if n == 0 or not p.value:
                return np.zeros(0, np.int32)
            return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int)), shape=(n,)).copy()

        self.n1 = n1.value
        self.ptr1 = view(ptrs[0], n1.value + 1)
        self.ptr2 = view(ptrs[1], npart.value + 1)
        self.id = view(ptrs[2], nid.value)
        self.type = view(ptrs[3], nid.value)
        self.ker_begin = view(ptrs[4], 2 * npart.value) if hk.value else None
        st = (C.c_double * 5)()
        check(L.tf_schedule_stats(self._h, st))
        self.stats = np.array(st[:], dtype=np.float64)

    @classmethod
    def from_arrays(cls, n1, ptr1, ptr2, ids, types, ker_begin=None):
        h = C.c_void_p()
        a = [_i32(x) for x in (ptr1, ptr2, ids, types)]
        k = _i32(ker_begin) if ker_begin is not None else None
        check(_lib.lib().tf_schedule_from_arrays(int(n1), a[0].ctypes.data, a[1].ctypes.data, a[2].ctypes.data,
                                                 a[3].ctypes.data, k.ctypes.data if k is not None else None,
                                                 C.byref(h)))
        return cls(h.value)

    def serialize(self) -> np.ndarray:
        n = C.c_size_t()
        check(_lib.lib().tf_schedule_serialized_size(self._h, C.byref(n)))
        buf = np.zeros(n.value, np.int32)
        check(_lib.lib().tf_schedule_serialize(self._h, buf.ctypes.data, n.value))
        return buf

    @classmethod
    def deserialize(cls, buf: np.ndarray):
        b = _i32(buf)
        h = C.c_void_p()
        check(_lib.lib().tf_schedule_deserialize(b.ctypes.data, b.shape[0], C.byref(h)))
        return cls(h.value)

    @property
    def num_partitions(self):
        return int(self.ptr1[self.n1])

    @property
    def fused_rows(self):
        return int(self.stats[0])

    def __del__(self):
        try:
            if self._h:
                _lib.lib().tf_schedule_free(self._h)
                self._h = None
        except Exception:
            pass


def inspector(A: CSRMatrix, NumThreads: int, params: ScheduleParameters | None = None, **kw) -> FusedSchedule:
    """FusedSchedule inspector(CSRMatrix A, int NumThreads) -- README.md:25.

    The README form takes no tile parameters although every in-tree inspector needs them
    (Fusion_Defs.h:21-33); ``params`` (or keyword overrides of its fields) selects the reference
    inspector and its arguments.  The returned arrays are bit-identical to the reference's."""
    p = params or ScheduleParameters()
    p = ScheduleParameters(**{**p.__dict__, "num_threads": int(NumThreads), **kw})
    sp = _lib.SchedParams(p.kind, p.num_threads, p.iter_per_partition, p.tile_m, p.b_cols, p.c_cols, p.data_size)
    h = C.c_void_p()
    check(_lib.lib().tf_inspect(A.M, A.Ap.ctypes.data, A.Ai.ctypes.data, C.byref(sp), C.byref(h)))
    return FusedSchedule(h.value, p)


def _stream_ptr():
    import torch
    return torch.cuda.current_stream().cuda_stream


class Plan:
    """Device-resident operators plus the executor's item list for one chain.

    chain: "spmm_spmm" (A, optional B, n_cols), "gemm_spmm" (A, k, n_cols) or "sddmm_spmm" (A, kq, nv).
    """

    def __init__(self, chain: str, A: CSRMatrix, *, B: CSRMatrix | None = None, k: int = 0, n_cols: int = 0,
                 mode: int = MODE_STREAM, schedule: FusedSchedule | None = None, rows_per_block: int = 0,
                 ring_bytes: int = 0, slack_blocks: int = -1, ctas_per_sm: int = 0, halo_rows: int = 0,
                 boundary_rows=None, tile_slots: int = 0, tile_max_bz: int = 0, tensor_cores: int = 0,
                 tile_double_buffer: int = 0, tile_pipeline: int = 0, lattice_march: int = 0):
        L = _lib.lib()
        self.chain, self.A, self.B = chain, A, B
        self.n_cols, self.k = int(n_cols), int(k)
        br = _i32(boundary_rows) if boundary_rows is not None and len(boundary_rows) else None
        o = _lib.PlanOpts(mode, rows_per_block, ring_bytes, slack_blocks, ctas_per_sm, halo_rows,
                          0 if br is None else br.shape[0], None if br is None else br.ctypes.data,
                          tile_slots, tile_max_bz, tile_double_buffer, tensor_cores, tile_pipeline, lattice_march)
        h = C.c_void_p()
        ca = A._c()
        sh = schedule._h if schedule is not None else None
        if chain == "spmm_spmm":
            cb = B._c() if B is not None else None
            check(L.tf_plan_spmm_spmm(C.byref(ca), C.byref(cb) if cb is not None else None, self.n_cols,
                                      C.byref(o), sh, C.byref(h)))
        elif chain == "gemm_spmm":
            check(L.tf_plan_gemm_spmm(C.byref(ca), self.k, self.n_cols, C.byref(o), sh, C.byref(h)))
        elif chain == "sddmm_spmm":
            check(L.tf_plan_sddmm_spmm(C.byref(ca), self.k, self.n_cols, C.byref(o), C.byref(h)))
        else:
            raise ValueError(f"unknown chain {chain!r}")
        self._h = h
        self._schedule = schedule  # keep alive

    @classmethod
    def adopt(cls, native_chain):
        """A view of the device plan inside a multi-GPU chain (distributed.NativeRankChain), for info() and status();
        the chain keeps ownership."""
        p = cls.__new__(cls)
        p._h = C.c_void_p(_lib.lib().tf_multi_plan_handle(native_chain._h))
        p._borrowed = True
        p._schedule = None
        return p

    # -- information ---------------------------------------------------------
    def info(self) -> dict:
        a = (C.c_longlong * 8)()
        check(_lib.lib().tf_plan_info(self._h, a))
        keys = ["items", "producer_blocks", "consumer_blocks", "ring_rows", "grid", "threads", "launches",
                "intermediate_rows"]
        return dict(zip(keys, [int(x) for x in a]))

    def status(self, stream: int | None = None) -> None:
        """Waits for the plan's work and raises if a bounded in-kernel wait ran out."""
        check(_lib.lib().tf_plan_status(self._h, stream if stream is not None else _stream_ptr()))

    def tile_info(self) -> dict:
        """Brick shape and tile count of the gather tiles of the first and second operator."""
        a = (C.c_int * 8)()
        check(_lib.lib().tf_plan_tile_info(self._h, a))
        return {"producer": tuple(a[0:4]), "consumer": tuple(a[4:8])}

    def set_wait_limit(self, polls: int) -> None:
        check(_lib.lib().tf_plan_set_wait_limit(self._h, int(polls)))

    def exchange_buffers(self):
        """(send_ptr, send_rows, halo_ptr, halo_rows) of the halo exchange."""
        sp, hp = C.c_void_p(), C.c_void_p()
        sr, hr = C.c_longlong(), C.c_longlong()
        check(_lib.lib().tf_plan_exchange_buffers(self._h, C.byref(sp), C.byref(sr), C.byref(hp), C.byref(hr)))
        return sp.value, sr.value, hp.value, hr.value

    # -- device executors (torch CUDA tensors) -------------------------------
    def spmm_spmm(self, Cd, Dd, stream=None):
        check(_lib.lib().tf_exec_spmm_spmm(self._h, Cd.data_ptr(), Dd.data_ptr(),
                                           stream if stream is not None else _stream_ptr()))

    def gemm_spmm(self, Bd, Wd, Dd, w_transposed=False, relu=False, stream=None):
        check(_lib.lib().tf_exec_gemm_spmm(self._h, Bd.data_ptr(), Wd.data_ptr(), int(w_transposed), int(relu),
                                           Dd.data_ptr(), stream if stream is not None else _stream_ptr()))

    def sddmm_spmm(self, Qd, Kd, Vd, Dd, stream=None):
        check(_lib.lib().tf_exec_sddmm_spmm(self._h, Qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), Dd.data_ptr(),
                                            stream if stream is not None else _stream_ptr()))

    def phase(self, phase, in0, in1=None, out=None, w_transposed=False, relu=False, stream=None):
        check(_lib.lib().tf_exec_phase(self._h, int(phase), in0.data_ptr(), in1.data_ptr() if in1 is not None else None,
                                       int(w_transposed), int(relu), out.data_ptr() if out is not None else None,
                                       stream if stream is not None else _stream_ptr()))

    # -- host executors (numpy) ------------------------------------------------
    def spmm_spmm_host(self, Ch: np.ndarray, Dh: np.ndarray):
        check(_lib.lib().tf_spmm_spmm_host(self._h, Ch.ctypes.data, Dh.ctypes.data))

    def gemm_spmm_host(self, Bh, Wh, Dh, w_transposed=False, relu=False):
        check(_lib.lib().tf_gemm_spmm_host(self._h, Bh.ctypes.data, Wh.ctypes.data, int(w_transposed), int(relu),
                                           Dh.ctypes.data))

    def sddmm_spmm_host(self, Qh, Kh, Vh, Dh):
        check(_lib.lib().tf_sddmm_spmm_host(self._h, Qh.ctypes.data, Kh.ctypes.data, Vh.ctypes.data, Dh.ctypes.data))

    def close(self):
        if getattr(self, "_h", None):
            if not getattr(self, "_borrowed", False):
                _lib.lib().tf_plan_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_plan_cache: dict = {}


def _cached_plan(key, make):
    p = _plan_cache.get(key)
    if p is None:
        if len(_plan_cache) >= 8:
            _plan_cache.pop(next(iter(_plan_cache))).close()
        p = _plan_cache[key] = make()
    return p


def _mode_for(schedule, mode):
    if mode is not None:
        return mode
    return MODE_STREAM


def spMMSpMMExecutor(A: CSRMatrix, B: CSRMatrix, C_: Matrix, D: Matrix, schedule: FusedSchedule | None,
                     NumThreads: int = 1, mode: int | None = None):
    """D = A * (B * C), A and B sparse -- README.md:31.  ``NumThreads`` is kept for source compatibility and
    does not affect the GPU executor.  mode=MODE_SCHEDULE follows ``schedule`` tile by tile as the reference
    executor does; the default streams the chain through the L2-resident ring (same result)."""
    if C_.N != D.N or D.M != A.M or C_.M != B.N or B.M != A.N:
        raise ValueError("spMMSpMMExecutor: shapes do not chain")
    if C_.on_device != D.on_device:
        raise ValueError("spMMSpMMExecutor: C and D must both be host or both be device data")
    m = _mode_for(schedule, mode)
    same = B is A
    key = ("ss", A.fingerprint(), B.fingerprint(), C_.N, m, id(schedule) if m == MODE_SCHEDULE else 0)
    plan = _cached_plan(key, lambda: Plan("spmm_spmm", A, B=None if same else B, n_cols=C_.N, mode=m,
                                          schedule=schedule if m == MODE_SCHEDULE else None))
    if C_.on_device:
        plan.spmm_spmm(C_.Data, D.Data)
    else:
        plan.spmm_spmm_host(C_.Data, D.Data)
    return D


def geMMSpMMExecutor(A: CSRMatrix, B: Matrix, C_: Matrix, D: Matrix, schedule: FusedSchedule | None,
                     NumThreads: int = 1, mode: int | None = None, w_transposed: bool = False, relu: bool = False):
    """D = A * (B * C), B and C dense -- README.md:32.  C is K x N (the layout of
    forwardForOneLayerFusedParallelSeparatedVectorizedSP) or, with w_transposed, N x K (the torch binding's)."""
    k = B.N
    n = C_.M if w_transposed else C_.N
    if (C_.N if w_transposed else C_.M) != k or D.N != n or D.M != A.M or B.M != A.N:
        raise ValueError("geMMSpMMExecutor: shapes do not chain")
    if not (B.on_device == C_.on_device == D.on_device):
        raise ValueError("geMMSpMMExecutor: B, C and D must all be host or all be device data")
    m = _mode_for(schedule, mode)
    key = ("gs", A.fingerprint(), k, n, m, id(schedule) if m == MODE_SCHEDULE else 0)
    plan = _cached_plan(key, lambda: Plan("gemm_spmm", A, k=k, n_cols=n, mode=m,
                                          schedule=schedule if m == MODE_SCHEDULE else None))
    if B.on_device:
        plan.gemm_spmm(B.Data, C_.Data, D.Data, w_transposed, relu)
    else:
        plan.gemm_spmm_host(B.Data, C_.Data, D.Data, w_transposed, relu)
    return D


def sddmmSpMMExecutor(A: CSRMatrix, Q: Matrix, K: Matrix, V: Matrix, D: Matrix):
    """D = (A .* (Q K^T)) V.  The reference has the SDDMM half only (codegen/triton/sddmm.py:173-184)."""
    if Q.N != K.N or Q.M != A.M or K.M != A.N or V.M != A.N or D.M != A.M or D.N != V.N:
        raise ValueError("sddmmSpMMExecutor: shapes do not chain")
    key = ("sd", A.fingerprint(), Q.N, V.N)
    plan = _cached_plan(key, lambda: Plan("sddmm_spmm", A, k=Q.N, n_cols=V.N))
    if Q.on_device:
        plan.sddmm_spmm(Q.Data, K.Data, V.Data, D.Data)
    else:
        plan.sddmm_spmm_host(Q.Data, K.Data, V.Data, D.Data)
    return D


def gcn_forward(A: CSRMatrix, X, W1, W2, plans=None):
    """Two-layer GCN forward, out = A (relu(A (X W1^T)) W2^T), weights stored [out, in]
    (binding-project/gcn-e2e-training/FusedGCNModule.py:14-18).  X, W1, W2: CUDA torch tensors."""
    import torch
    n = A.M
    hid, out = W1.shape[0], W2.shape[0]
    if plans is None:
        plans = (Plan("gemm_spmm", A, k=X.shape[1], n_cols=hid), Plan("gemm_spmm", A, k=hid, n_cols=out))
    h1 = torch.empty((n, hid), device=X.device, dtype=torch.float32)
    o = torch.empty((n, out), device=X.device, dtype=torch.float32)
    plans[0].gemm_spmm(X, W1, h1, w_transposed=True, relu=True)
    plans[1].gemm_spmm(h1, W2, o, w_transposed=True, relu=False)
    return o, plans


def plan_preview(A: CSRMatrix, B: CSRMatrix | None = None, *, producer_is_gemm=False, n_cols=128,
                 resident_ctas=592, mode=MODE_STREAM, rows_per_block=0, ring_bytes=0, slack_blocks=-1,
                 halo_rows=0, boundary_rows=None, tile_slots=0, tile_max_bz=0):
    """Host-only: the item list the stream executor would walk, as an (n, 8) int array
    {kind, block, row_begin, row_end, need, base, aux0, aux1}, plus an info dict."""
    br = _i32(boundary_rows) if boundary_rows is not None and len(boundary_rows) else None
    o = _lib.PlanOpts(mode, rows_per_block, ring_bytes, slack_blocks, 0, halo_rows,
                      0 if br is None else br.shape[0], None if br is None else br.ctypes.data, tile_slots, tile_max_bz, 0, 0, 0, 0)
    ca = A._c()
    cb = B._c() if B is not None else None
    items, n = C.c_void_p(), C.c_longlong()
    info = (C.c_longlong * 8)()
    check(_lib.lib().tf_plan_preview(C.byref(ca), C.byref(cb) if cb is not None else None, int(producer_is_gemm),
                                     int(n_cols), C.byref(o), int(resident_ctas), C.byref(items), C.byref(n), info))
    arr = np.ctypeslib.as_array(C.cast(items, C.POINTER(C.c_int)), shape=(max(n.value, 1) * 8,)).copy()
    _lib.lib().tf_free(items)
    keys = ["items", "producer_blocks", "consumer_blocks", "ring_rows", "phase1_begin", "phase2_begin", "end",
            "intermediate_rows"]
    return arr[:n.value * 8].reshape(-1, 8), dict(zip(keys, [int(x) for x in info]))


def tiling_preview(A: CSRMatrix, tile_slots=0, tile_max_bz=0):
    """Host-only: the gather tiles of operator A as (row_ptr, rows, halo_ptr, halo, info) or None."""
    ca = A._c()
    ptrs = [C.c_void_p() for _ in range(4)]
    n, info = C.c_int(), (C.c_int * 4)()
    check(_lib.lib().tf_tiling_preview(C.byref(ca), tile_slots, tile_max_bz, *[C.byref(p) for p in ptrs], C.byref(n), info))

    def take(p, count):
        arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int)), shape=(max(count, 1),)).copy()[:count]
        _lib.lib().tf_free(p)
        return arr
    if n.value == 0:
        for p in ptrs:
            _lib.lib().tf_free(p)
        return None
    row_ptr = take(ptrs[0], n.value + 1)
    halo_ptr_raw = ptrs[2]
    rows = take(ptrs[1], int(row_ptr[-1]))
    halo_ptr = take(halo_ptr_raw, n.value + 1)
    halo = take(ptrs[3], int(halo_ptr[-1]))
    return row_ptr, rows, halo_ptr, halo, dict(bx=info[0], by=info[1], bz=info[2], reuse=info[3] / 1000.0)


def lattice_preview(A: CSRMatrix, halo_rows=0, n_cols=128, ctas=148):
    """Host-only: operator A as a star stencil on a 3-D grid (what the plane-marching executor runs from), or None
    when the pattern is not one.  Returns dict(nx, ny, nz, ghost_lo, ghost_hi, classes, dict, patch_cls, items)."""
    ca = A._c()
    info = (C.c_int * 8)()
    d, pc, it = C.c_void_p(), C.c_void_p(), C.c_void_p()
    n = C.c_int()
    check(_lib.lib().tf_lattice_preview(C.byref(ca), int(halo_rows), int(n_cols), int(ctas), info, C.byref(d),
                                        C.byref(pc), C.byref(it), C.byref(n)))
    if not info[0]:
        return None
    nx, ny, nz, ncls = info[1], info[2], info[3], info[6]

    def take(p, ctype, count, dtype):
        arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(ctype)), shape=(max(count, 1),)).copy()[:count].astype(dtype)
        _lib.lib().tf_free(p)
        return arr
    dic = take(d, C.c_float, (ncls + 1) * 8, np.float32).reshape(ncls + 1, 8)
    pcl = take(pc, C.c_uint, nz * ((ny + 1) // 2) * ((nx + 1) // 2), np.uint32).reshape(nz, (ny + 1) // 2, (nx + 1) // 2)
    items = take(it, C.c_int, 6 * n.value, np.int32).reshape(-1, 6)
    return dict(nx=nx, ny=ny, nz=nz, ghost_lo=info[4], ghost_hi=info[5], classes=ncls, dict=dic, patch_cls=pcl,
                items=items)


def read_matrix(path: str, expand_symmetric: bool = True) -> CSRMatrix:
    """A sparse matrix file as a CSRMatrix: Matrix Market coordinate files (*.mtx) and the DLMC text format (*.smtx)
    -- the two formats the reference's drivers read (fusion/src/Fusion_Utils.cpp:205-272)."""
    m, n, nnz = C.c_int(), C.c_int(), C.c_longlong()
    ap, ai, ax = C.c_void_p(), C.c_void_p(), C.c_void_p()
    check(_lib.lib().tf_read_matrix(str(path).encode(), int(expand_symmetric), C.byref(m), C.byref(n), C.byref(nnz),
                                    C.byref(ap), C.byref(ai), C.byref(ax)))

    def take(p, ctype, count, dtype):
        a = np.ctypeslib.as_array(C.cast(p, C.POINTER(ctype)), shape=(max(count, 1),)).copy()[:count].astype(dtype)
        _lib.lib().tf_free(p)
        return a
    return CSRMatrix(m.value, n.value, take(ap, C.c_int, m.value + 1, np.int32), take(ai, C.c_int, nnz.value, np.int32),
                     take(ax, C.c_float, nnz.value, np.float32))


def read_dense_mtx(path: str) -> np.ndarray:
    """A dense matrix from a Matrix Market array file (fusion/src/Fusion_Utils.cpp:274-283), row-major float32."""
    r, c, d = C.c_int(), C.c_int(), C.c_void_p()
    check(_lib.lib().tf_read_dense_mtx(str(path).encode(), C.byref(r), C.byref(c), C.byref(d)))
    a = np.ctypeslib.as_array(C.cast(d, C.POINTER(C.c_float)), shape=(r.value * c.value,)).copy().reshape(r.value, c.value)
    _lib.lib().tf_free(d)
    return a


def _take(p, ctype, count, dtype):
    a = np.ctypeslib.as_array(C.cast(p, C.POINTER(ctype)), shape=(max(count, 1),)).copy()[:count].astype(dtype)
    _lib.lib().tf_free(p)
    return a


def unfused_csr(schedule: FusedSchedule, A: CSRMatrix):
    """(UFAp, UFAi, UFAx): the second-wave rows of a schedule as their own CSR, in schedule order
    (createUnfusedData, fusion/example/SpMM_SpMM_SP_Demo_Utils.h:600-636)."""
    p, ci, x, n = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_int()
    check(_lib.lib().tf_schedule_unfused_csr(schedule._h, A.M, A.Ap.ctypes.data, A.Ai.ctypes.data, A.Ax.ctypes.data,
                                             C.byref(p), C.byref(ci), C.byref(x), C.byref(n)))
    ap = _take(p, C.c_int, n.value + 1, np.int32)
    nnz = int(ap[-1])
    return ap, _take(ci, C.c_int, nnz, np.int32), _take(x, C.c_float, nnz, np.float32)


def reordered_adjacency(schedule: FusedSchedule, A: CSRMatrix):
    """(Ap, Ai, Ax, L2Ptr, NewMixPtr): A's rows in the order the schedule's second loop visits them
    (createReorderedAdj, fusion/gcn/SingleLayer/GCN_Single_Layer_SP_Demo_Utils.h:618-653)."""
    ptrs = [C.c_void_p() for _ in range(5)]
    n = C.c_int()
    check(_lib.lib().tf_schedule_reordered_adj(schedule._h, A.M, A.Ap.ctypes.data, A.Ai.ctypes.data, A.Ax.ctypes.data,
                                               *[C.byref(q) for q in ptrs], C.byref(n)))
    return (_take(ptrs[0], C.c_int, A.M + 1, np.int32), _take(ptrs[1], C.c_int, A.nnz, np.int32),
            _take(ptrs[2], C.c_float, A.nnz, np.float32), _take(ptrs[3], C.c_int, A.M, np.int32),
            _take(ptrs[4], C.c_int, n.value, np.int32))


def rcm_order(A: CSRMatrix) -> np.ndarray:
    """Reverse Cuthill-McKee ordering of A's symmetrised pattern: perm[new] = old."""
    perm = np.empty(A.M, np.int32)
    check(_lib.lib().tf_rcm_order(A.M, A.Ap.ctypes.data, A.Ai.ctypes.data, perm.ctypes.data))
    return perm


def permute(A: CSRMatrix, perm) -> CSRMatrix:
    """P A P^T for perm[new] = old, columns sorted."""
    perm = _i32(perm)
    ap, ai, ax = np.empty(A.M + 1, np.int32), np.empty(A.nnz, np.int32), np.empty(A.nnz, np.float32)
    check(_lib.lib().tf_permute_csr(A.M, A.Ap.ctypes.data, A.Ai.ctypes.data, A.Ax.ctypes.data, perm.ctypes.data,
                                    ap.ctypes.data, ai.ctypes.data, ax.ctypes.data))
    return CSRMatrix(A.M, A.N, ap, ai, ax)
