"""ctypes bindings of the two CPU oracles (test infrastructure, see oracle/__init__.py)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")


def build(ref: bool = True) -> None:
    """Compile the restatement and, where the reference tree exists, the reference itself."""
    subprocess.run(["make", "-C", _HERE, "oracle"], check=True, capture_output=True)
    ref_root = os.environ.get("TF_REFERENCE_ROOT", "/root/reference")
    if ref and os.path.isdir(os.path.join(ref_root, "fusion", "src")):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={ref_root}"], check=True, capture_output=True)


@dataclass
class Schedule:
    """Reference-format schedule (sym_lib::MultiDimensionalSet) as numpy arrays."""
    n1: int
    ptr1: np.ndarray
    ptr2: np.ndarray
    id: np.ndarray
    type: np.ndarray
    ker_begin: np.ndarray | None
    stats: np.ndarray  # fused nodes, fused nnz, tile mean, tile std, partitions

    def same_arrays(self, other: "Schedule") -> bool:
        if self.n1 != other.n1:
            return False
        for a, b in ((self.ptr1, other.ptr1), (self.ptr2, other.ptr2), (self.id, other.id),
                     (self.type, other.type)):
            if a.shape != b.shape or not np.array_equal(a, b):
                return False
        if (self.ker_begin is None) != (other.ker_begin is None):
            return False
        return self.ker_begin is None or np.array_equal(self.ker_begin, other.ker_begin)


def _pull(lib, prefix, h) -> Schedule:
    n1, npart, nid, hk = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    getattr(lib, prefix + "sched_dims")(h, C.byref(n1), C.byref(npart), C.byref(nid), C.byref(hk))
    ptr1 = np.zeros(n1.value + 1, np.int32)
    ptr2 = np.zeros(npart.value + 1, np.int32)
    ids = np.zeros(max(nid.value, 1), np.int32)
    typ = np.zeros(max(nid.value, 1), np.int32)
    ker = np.zeros(max(2 * npart.value, 1), np.int32)
    stats = np.zeros(8, np.float64)
    getattr(lib, prefix + "sched_copy")(h, ptr1, ptr2, ids, typ, ker, stats)
    getattr(lib, prefix + "sched_free")(h)
    return Schedule(n1.value, ptr1, ptr2, ids[:nid.value], typ[:nid.value],
                    ker[:2 * npart.value] if hk.value else None, stats)


def _decl_sched(lib, prefix):
    getattr(lib, prefix + "sched_dims").argtypes = [C.c_void_p] + [C.POINTER(C.c_int)] * 4
    getattr(lib, prefix + "sched_dims").restype = None
    getattr(lib, prefix + "sched_copy").argtypes = [C.c_void_p, _i32p, _i32p, _i32p, _i32p, _i32p, _f64p]
    getattr(lib, prefix + "sched_copy").restype = None
    getattr(lib, prefix + "sched_free").argtypes = [C.c_void_p]
    getattr(lib, prefix + "sched_free").restype = None


class Oracle:
    """The plain-C restatement (oracle/tf_oracle.c)."""

    def __init__(self):
        path = os.path.join(_HERE, "libtf_oracle.so")
        if not os.path.exists(path):
            build(ref=False)
        L = self.lib = C.CDLL(path)
        _decl_sched(L, "orc_")
        L.orc_inspect_fixed.argtypes = [C.c_int, _i32p, _i32p, C.c_int, C.c_int]
        L.orc_inspect_fixed.restype = C.c_void_p
        L.orc_inspect_variable.argtypes = [C.c_int, C.c_int, _i32p, _i32p] + [C.c_int] * 5
        L.orc_inspect_variable.restype = C.c_void_p
        L.orc_spmm_csr.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, _f32p]
        L.orc_spmm_csr.restype = None
        L.orc_spmm_spmm_fused.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p, _f32p,
                                          _f32p, _f32p, _f32p, C.c_int, _i32p, _i32p, _i32p, _i32p]
        L.orc_spmm_spmm_fused.restype = None
        L.orc_gemm_spmm_fused.argtypes = [C.c_int, _i32p, _i32p, _f32p, C.c_int, C.c_int, _f32p, _f32p,
                                          C.c_int, _f32p, _f32p, C.c_int, _i32p, _i32p, _i32p, _i32p]
        L.orc_gemm_spmm_fused.restype = None
        L.orc_sddmm_spmm.argtypes = [C.c_int, _i32p, _i32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p,
                                     C.c_void_p, _f32p]
        L.orc_sddmm_spmm.restype = None
        L.orc_gcn_layer.argtypes = [C.c_int, _i32p, _i32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, C.c_int,
                                    _f32p, _f32p]
        L.orc_gcn_layer.restype = None
        L.orc_chain_f64.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, C.c_int, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_int, C.c_void_p, _f32p, _f64p, _f64p]
        L.orc_chain_f64.restype = None
        L.orc_sddmm_spmm_f64.argtypes = [C.c_int, _i32p, _i32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p,
                                         _f64p]
        L.orc_sddmm_spmm_f64.restype = None

    # -- inspectors ------------------------------------------------------
    def inspect_fixed(self, ap, ai, threads, iter_per_part) -> Schedule:
        h = self.lib.orc_inspect_fixed(len(ap) - 1, ap, ai, threads, iter_per_part)
        return _pull(self.lib, "orc_", h)

    def inspect_variable(self, kind, ap, ai, threads, tile_m, bcol, ccol=0, data_size=4):
        """kind 2 = SpMM-SpMM both wavefronts, 3 = GeMM-SpMM, 4 = SpMM-SpMM, wave 2 split by threads.
        Returns None where the reference would divide by zero or never terminate."""
        h = self.lib.orc_inspect_variable(kind, len(ap) - 1, ap, ai, threads, tile_m, bcol, ccol, data_size)
        return _pull(self.lib, "orc_", h) if h else None

    # -- executors -------------------------------------------------------
    def spmm(self, ap, ai, ax, b):
        out = np.zeros((len(ap) - 1, b.shape[1]), np.float32)
        self.lib.orc_spmm_csr(len(ap) - 1, b.shape[1], ap, ai, ax, np.ascontiguousarray(b), out)
        return out

    def spmm_spmm(self, a, b, c, sched: Schedule):
        """D = A*(B*C); a, b are (Ap, Ai, Ax) triples; B rows are the type-0 (first) loop."""
        m, n = len(a[0]) - 1, c.shape[1]
        d = np.zeros((m, n), np.float32)
        ac = np.zeros((m, n), np.float32)
        self.lib.orc_spmm_spmm_fused(m, n, b[0], b[1], b[2], a[0], a[1], a[2], np.ascontiguousarray(c), d, ac,
                                     sched.n1, sched.ptr1, sched.ptr2, sched.id, sched.type)
        return d, ac

    def gemm_spmm(self, a, feat, w, sched: Schedule, w_transposed=False):
        m, k = feat.shape
        n = w.shape[0] if w_transposed else w.shape[1]
        d = np.zeros((m, n), np.float32)
        tmp = np.zeros((m, n), np.float32)
        self.lib.orc_gemm_spmm_fused(m, a[0], a[1], a[2], k, n, np.ascontiguousarray(feat),
                                     np.ascontiguousarray(w), int(w_transposed), d, tmp, sched.n1,
                                     sched.ptr1, sched.ptr2, sched.ker_begin, sched.id)
        return d, tmp

    def sddmm_spmm(self, a, q, k, v, want_s=False):
        m = len(a[0]) - 1
        d = np.zeros((m, v.shape[1]), np.float32)
        s = np.zeros(len(a[1]), np.float32) if want_s else None
        self.lib.orc_sddmm_spmm(m, a[0], a[1], a[2], q.shape[1], v.shape[1], np.ascontiguousarray(q),
                                np.ascontiguousarray(k), np.ascontiguousarray(v),
                                s.ctypes.data if want_s else None, d)
        return (d, s) if want_s else d

    def gcn_layer(self, a, x, w, relu):
        m = len(a[0]) - 1
        out = np.zeros((m, w.shape[0]), np.float32)
        tmp = np.zeros((m, w.shape[0]), np.float32)
        self.lib.orc_gcn_layer(m, a[0], a[1], a[2], x.shape[1], w.shape[0], np.ascontiguousarray(x),
                               np.ascontiguousarray(w), int(relu), tmp, out)
        return out

    def gcn2(self, a, x, w1, w2):
        return self.gcn_layer(a, self.gcn_layer(a, x, w1, True), w2, False)

    def chain_f64(self, a, c, b_sparse=None, b_dense=None):
        m, n = len(a[0]) - 1, c.shape[1]
        d = np.zeros((m, n), np.float64)
        tmp = np.zeros((m, n), np.float64)
        if b_sparse is not None:
            self.lib.orc_chain_f64(m, n, a[0], a[1], a[2], 1, b_sparse[0].ctypes.data, b_sparse[1].ctypes.data,
                                   b_sparse[2].ctypes.data, 0, None, np.ascontiguousarray(c), tmp, d)
        else:
            bd = np.ascontiguousarray(b_dense)
            self.lib.orc_chain_f64(m, n, a[0], a[1], a[2], 0, None, None, None, bd.shape[1], bd.ctypes.data,
                                   np.ascontiguousarray(c), tmp, d)
        return d

    def sddmm_spmm_f64(self, a, q, k, v):
        d = np.zeros((len(a[0]) - 1, v.shape[1]), np.float64)
        self.lib.orc_sddmm_spmm_f64(len(a[0]) - 1, a[0], a[1], a[2], q.shape[1], v.shape[1],
                                    np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), d)
        return d


class Ref:
    """The unmodified reference compiled in place (oracle/_ref/libtf_ref.so)."""

    PATH = os.path.join(_HERE, "_ref", "libtf_ref.so")
    PATH_AVX512 = os.path.join(_HERE, "_ref", "libtf_ref_avx512.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    @classmethod
    def avx512_available(cls) -> bool:
        """The AVX-512 build exists and this host's CPU can run it."""
        if not os.path.exists(cls.PATH_AVX512):
            return False
        try:
            with open("/proc/cpuinfo") as f:
                return any("avx512f" in line for line in f if line.startswith("flags"))
        except OSError:
            return False

    def __init__(self, use_mkl_sgemm: bool = True, avx512: bool = False):
        L = self.lib = C.CDLL(self.PATH_AVX512 if avx512 else self.PATH)
        L.tf_ref_has_avx512.restype = C.c_int
        self.has_avx512 = bool(L.tf_ref_has_avx512())
        L.tf_ref_normalize_adjacency.argtypes = [C.c_int, _i32p, _i32p, _f64p]
        L.tf_ref_normalize_adjacency.restype = C.c_int
        _decl_sched(L, "tf_ref_")
        L.tf_ref_inspect.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p] + [C.c_int] * 6
        L.tf_ref_inspect.restype = C.c_void_p
        L.tf_ref_spmm_csr.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, _f32p, C.c_int]
        L.tf_ref_spmm_csr.restype = None
        L.tf_ref_spmm_spmm_fused.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p,
                                             _f32p, _f32p, _f32p, _f32p, C.c_int, _i32p, _i32p, _i32p, _i32p,
                                             C.c_int]
        L.tf_ref_spmm_spmm_fused.restype = None
        L.tf_ref_gemm_spmm_fused.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, C.c_int, C.c_int, _f32p,
                                             _f32p, _f32p, _f32p, C.c_int, C.c_int, _i32p, _i32p, _i32p, _i32p]
        L.tf_ref_gemm_spmm_fused.restype = None
        L.tf_ref_gemm_spmm_unfused.argtypes = [C.c_int, _i32p, _i32p, _f32p, C.c_int, C.c_int, _f32p, _f32p,
                                               _f32p, _f32p, C.c_int]
        L.tf_ref_gemm_spmm_unfused.restype = None
        L.tf_ref_set_sgemm.argtypes = [C.c_void_p]
        L.tf_ref_has_sgemm.restype = C.c_int
        self.sgemm = "loop"
        if use_mkl_sgemm:
            try:  # MKL's Fortran sgemm_ as exported by torch's CPU library
                import torch
                tl = C.CDLL(os.path.join(os.path.dirname(torch.__file__), "lib", "libtorch_cpu.so"))
                L.tf_ref_set_sgemm(C.cast(tl.sgemm_, C.c_void_p))
                self._torch_lib = tl
                self.sgemm = "mkl(libtorch_cpu)"
            except Exception:  # keep the plain-loop fallback
                pass

    def inspect(self, kind, ap, ai, threads, iter_per_part=1, tile_m=1, bcol=1, ccol=1, data_size=4):
        h = self.lib.tf_ref_inspect(kind, len(ap) - 1, len(ai), ap, ai, threads, iter_per_part, tile_m, bcol,
                                    ccol, data_size)
        return _pull(self.lib, "tf_ref_", h)

    def normalize_adjacency(self, ap, ai, ax):
        """GnnTensorSpInputs::normalizeAdjacencyMatrix on a copy of the values (doubles, as the reference's
        CSR holds them); returns the normalised doubles."""
        x = np.ascontiguousarray(ax, dtype=np.float64).copy()
        if not self.lib.tf_ref_normalize_adjacency(len(ap) - 1, np.ascontiguousarray(ap, dtype=np.int32),
                                                   np.ascontiguousarray(ai, dtype=np.int32), x):
            raise RuntimeError("the reference's normalizeAdjacencyMatrix was not built into oracle/_ref")
        return x

    def layouts(self, kind, ap, ai, ax, threads, iter_per_part=1, tile_m=1, bcol=1, ccol=1):
        """(createUnfusedData arrays, createReorderedAdj arrays) of the reference for the schedule its own inspector
        `kind` makes: ((UFAp, UFAi, UFAx), (Ap, Ai, Ax, L2Ptr, NewMixPtr))."""
        L = self.lib
        m, nnz = len(ap) - 1, len(ai)
        h = L.tf_ref_inspect(kind, m, nnz, ap, ai, threads, iter_per_part, tile_m, bcol, ccol, 4)
        L.tf_ref_create_unfused_data.argtypes = [C.c_void_p, C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p, _f32p]
        L.tf_ref_create_reordered_adj.argtypes = [C.c_void_p, C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p, _f32p, _i32p, _i32p]
        ufp, ufi, ufx = np.zeros(m + 1, np.int32), np.zeros(max(nnz, 1), np.int32), np.zeros(max(nnz, 1), np.float32)
        rows = L.tf_ref_create_unfused_data(C.c_void_p(h), m, ap, ai, ax, ufp, ufi, ufx)
        if rows < 0:
            raise RuntimeError("the reference's layout builders were not built into oracle/_ref")
        rp, ri, rx = np.zeros(m + 1, np.int32), np.zeros(max(nnz, 1), np.int32), np.zeros(max(nnz, 1), np.float32)
        l2, mix = np.zeros(m, np.int32), np.zeros(4 * m + 8, np.int32)
        n_mix = L.tf_ref_create_reordered_adj(C.c_void_p(h), m, ap, ai, ax, rp, ri, rx, l2, mix)
        L.tf_ref_sched_free.argtypes = [C.c_void_p]
        L.tf_ref_sched_free(C.c_void_p(h))
        k = int(ufp[rows])
        return (ufp[:rows + 1], ufi[:k], ufx[:k]), (rp, ri[:nnz], rx[:nnz], l2, mix[:n_mix])

    def spmm(self, ap, ai, ax, b, threads=1):
        out = np.zeros((len(ap) - 1, b.shape[1]), np.float32)
        self.lib.tf_ref_spmm_csr(len(ap) - 1, b.shape[1], ap, ai, ax, np.ascontiguousarray(b), out, threads)
        return out

    def spmm_spmm(self, a, b, c, sched: Schedule, threads=1, variant=1, out=None):
        m, n = len(a[0]) - 1, c.shape[1]
        if out is None:
            d, ac = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)
        else:
            d, ac = out
        # reference argument order: first operator (type 0) then second (type 1)
        self.lib.tf_ref_spmm_spmm_fused(variant, m, n, b[0], b[1], b[2], a[0], a[1], a[2],
                                        np.ascontiguousarray(c), d, ac, sched.n1, sched.ptr1, sched.ptr2,
                                        sched.id, sched.type, threads)
        return d, ac

    def gemm_spmm(self, a, feat, w, sched: Schedule, threads=1, variant=1, out=None):
        m, k = feat.shape
        n = w.shape[1] if variant == 1 else w.shape[0]
        if out is None:
            d, tmp = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)
        else:
            d, tmp = out
        self.lib.tf_ref_gemm_spmm_fused(variant, m, a[0], a[1], a[2], k, n, np.ascontiguousarray(feat),
                                        np.ascontiguousarray(w), d, tmp, threads, sched.n1, sched.ptr1,
                                        sched.ptr2, sched.ker_begin, sched.id)
        return d, tmp

    def gemm_spmm_unfused(self, a, feat, w, threads=1):
        m, k = feat.shape
        n = w.shape[1]
        d, tmp = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)
        self.lib.tf_ref_gemm_spmm_unfused(m, a[0], a[1], a[2], k, n, np.ascontiguousarray(feat),
                                          np.ascontiguousarray(w), d, tmp, threads)
        return d
