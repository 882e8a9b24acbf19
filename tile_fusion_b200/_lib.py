"""ctypes view of the C ABI declared in include/tile_fusion_b200.h."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtilefusion_b200.so")

TF_OK, TF_ERR_ARG, TF_ERR_UNSUPPORTED, TF_ERR_CUDA, TF_ERR_TIMEOUT, TF_ERR_NOMEM = 0, -1, -2, -3, -4, -5
INSPECT_FIXED, INSPECT_VT_SPMM, INSPECT_VT_GEMM, INSPECT_VT_SPMM_THREADS = 1, 2, 3, 4
MODE_STREAM, MODE_SCHEDULE, MODE_UNFUSED = 0, 1, 2


class TileFusionError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"tile_fusion_b200 error {code}: {msg}")
        self.code = code


class SchedParams(C.Structure):
    _fields_ = [("kind", C.c_int), ("num_threads", C.c_int), ("iter_per_partition", C.c_int),
                ("tile_m", C.c_int), ("b_cols", C.c_int), ("c_cols", C.c_int), ("data_size", C.c_int)]


class Csr(C.Structure):
    _fields_ = [("m", C.c_int), ("n", C.c_int), ("ap", C.c_void_p), ("ai", C.c_void_p), ("ax", C.c_void_p)]


class PlanOpts(C.Structure):
    _fields_ = [("mode", C.c_int), ("rows_per_block", C.c_int), ("ring_bytes", C.c_int),
                ("slack_blocks", C.c_int), ("ctas_per_sm", C.c_int), ("halo_rows", C.c_int),
                ("n_boundary", C.c_int), ("boundary_rows", C.c_void_p), ("tile_slots", C.c_int),
                ("tile_max_bz", C.c_int), ("tile_double_buffer", C.c_int), ("tensor_cores", C.c_int),
                ("tile_pipeline", C.c_int), ("lattice_march", C.c_int), ("exchange", C.c_int)]


EXPORTS = [
    "tf_last_error", "tf_version", "tf_inspect", "tf_schedule_dims", "tf_schedule_arrays", "tf_schedule_stats",
    "tf_schedule_from_arrays", "tf_schedule_serialized_size", "tf_schedule_serialize", "tf_schedule_deserialize",
    "tf_schedule_free", "tf_plan_spmm_spmm", "tf_plan_gemm_spmm", "tf_plan_sddmm_spmm", "tf_plan_free",
    "tf_plan_info", "tf_plan_status", "tf_exec_spmm_spmm", "tf_exec_gemm_spmm", "tf_exec_sddmm_spmm",
    "tf_exec_phase", "tf_plan_intermediate", "tf_plan_exchange_buffers", "tf_spmm_spmm_host", "tf_gemm_spmm_host",
    "tf_sddmm_spmm_host", "tf_spmm_dev", "tf_fill_uniform", "tf_fill_normal", "tf_plan_preview", "tf_free", "tf_plan_set_wait_limit", "tf_tiling_preview", "tf_plan_tile_info", "tf_spmm_spmm_noalloc",
    "tf_noalloc_max_floats", "tf_gemm_tc_dev", "tf_lattice_preview", "tf_comm_unique_id", "tf_comm_create",
    "tf_comm_from_nccl", "tf_comm_free", "tf_multi_plan", "tf_multi_free", "tf_multi_info", "tf_multi_plan_handle",
    "tf_multi_exec", "tf_multi_status", "tf_multi_trace", "tf_partition_layout", "tf_read_matrix", "tf_read_dense_mtx",
    "tf_schedule_unfused_csr", "tf_schedule_reordered_adj", "tf_rcm_order", "tf_permute_csr",
]

_lib = None


def lib() -> C.CDLL:
    """Loads the CUDA library; there is no fallback when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m tile_fusion_b200.build` "
                          "(needs nvcc); this package has no CPU fallback")
    L = C.CDLL(LIB_PATH)
    vp, ip, i = C.c_void_p, C.POINTER(C.c_int), C.c_int
    L.tf_last_error.restype = C.c_char_p
    L.tf_version.restype = C.c_char_p
    L.tf_inspect.argtypes = [i, vp, vp, C.POINTER(SchedParams), C.POINTER(vp)]
    L.tf_schedule_dims.argtypes = [vp, ip, ip, ip, ip]
    L.tf_schedule_arrays.argtypes = [vp] + [C.POINTER(vp)] * 5
    L.tf_schedule_stats.argtypes = [vp, C.POINTER(C.c_double)]
    L.tf_schedule_from_arrays.argtypes = [i, vp, vp, vp, vp, vp, C.POINTER(vp)]
    L.tf_schedule_serialized_size.argtypes = [vp, C.POINTER(C.c_size_t)]
    L.tf_schedule_serialize.argtypes = [vp, vp, C.c_size_t]
    L.tf_schedule_deserialize.argtypes = [vp, C.c_size_t, C.POINTER(vp)]
    L.tf_schedule_free.argtypes = [vp]
    L.tf_schedule_free.restype = None
    L.tf_plan_spmm_spmm.argtypes = [C.POINTER(Csr), C.POINTER(Csr), i, C.POINTER(PlanOpts), vp, C.POINTER(vp)]
    L.tf_plan_gemm_spmm.argtypes = [C.POINTER(Csr), i, i, C.POINTER(PlanOpts), vp, C.POINTER(vp)]
    L.tf_plan_sddmm_spmm.argtypes = [C.POINTER(Csr), i, i, C.POINTER(PlanOpts), C.POINTER(vp)]
    L.tf_plan_free.argtypes = [vp]
    L.tf_plan_free.restype = None
    L.tf_plan_info.argtypes = [vp, C.POINTER(C.c_longlong)]
    L.tf_plan_status.argtypes = [vp, vp]
    L.tf_exec_spmm_spmm.argtypes = [vp, vp, vp, vp]
    L.tf_exec_gemm_spmm.argtypes = [vp, vp, vp, i, i, vp, vp]
    L.tf_exec_sddmm_spmm.argtypes = [vp, vp, vp, vp, vp, vp]
    L.tf_exec_phase.argtypes = [vp, i, vp, vp, i, i, vp, vp]
    L.tf_plan_intermediate.argtypes = [vp, C.POINTER(vp), C.POINTER(C.c_longlong), ip]
    L.tf_plan_exchange_buffers.argtypes = [vp, C.POINTER(vp), C.POINTER(C.c_longlong), C.POINTER(vp),
                                           C.POINTER(C.c_longlong)]
    L.tf_spmm_spmm_host.argtypes = [vp, vp, vp]
    L.tf_gemm_spmm_host.argtypes = [vp, vp, vp, i, i, vp]
    L.tf_sddmm_spmm_host.argtypes = [vp, vp, vp, vp, vp]
    L.tf_spmm_dev.argtypes = [vp, vp, vp, i, vp, i, vp, vp]
    L.tf_fill_uniform.argtypes = [vp, C.c_longlong, C.c_ulonglong, C.c_longlong, vp]
    L.tf_fill_normal.argtypes = [vp, C.c_longlong, C.c_ulonglong, C.c_longlong, C.c_float, vp]
    L.tf_plan_preview.argtypes = [C.POINTER(Csr), C.POINTER(Csr), i, i, C.POINTER(PlanOpts), i, C.POINTER(vp),
                                  C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]
    L.tf_free.argtypes = [vp]
    L.tf_plan_set_wait_limit.argtypes = [vp, i]
    L.tf_tiling_preview.argtypes = [C.POINTER(Csr), i, i] + [C.POINTER(vp)] * 4 + [ip, ip]
    L.tf_plan_tile_info.argtypes = [vp, ip]
    L.tf_spmm_spmm_noalloc.argtypes = [vp, vp, vp, i, vp, i, vp, vp]
    L.tf_noalloc_max_floats.restype = C.c_longlong
    L.tf_gemm_tc_dev.argtypes = [vp, vp, i, i, i, i, vp, vp]
    L.tf_free.restype = None
    ll = C.c_longlong
    L.tf_comm_unique_id.argtypes = [vp]
    L.tf_comm_create.argtypes = [vp, i, i, C.POINTER(vp)]
    L.tf_comm_from_nccl.argtypes = [vp, i, i, C.POINTER(vp)]
    L.tf_comm_free.argtypes = [vp]
    L.tf_comm_free.restype = None
    L.tf_multi_plan.argtypes = [vp, i, ll, ll, vp, vp, vp, i, i, C.POINTER(PlanOpts), C.POINTER(vp)]
    L.tf_multi_free.argtypes = [vp]
    L.tf_multi_free.restype = None
    L.tf_multi_info.argtypes = [vp, C.POINTER(ll)]
    L.tf_multi_plan_handle.argtypes = [vp]
    L.tf_multi_plan_handle.restype = vp
    L.tf_multi_exec.argtypes = [vp, vp, vp, i, i, vp, vp]
    L.tf_multi_status.argtypes = [vp, vp]
    L.tf_multi_trace.argtypes = [vp, C.c_int, C.POINTER(C.c_float)]
    L.tf_partition_layout.argtypes = [i, i, vp, vp, vp, C.POINTER(vp), C.POINTER(ll), C.POINTER(vp), ip, C.POINTER(vp), ip]
    L.tf_schedule_unfused_csr.argtypes = [vp, i, vp, vp, vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), ip]
    L.tf_schedule_reordered_adj.argtypes = [vp, i, vp, vp, vp] + [C.POINTER(vp)] * 5 + [ip]
    L.tf_rcm_order.argtypes = [i, vp, vp, vp]
    L.tf_permute_csr.argtypes = [i, vp, vp, vp, vp, vp, vp, vp]
    L.tf_read_matrix.argtypes = [C.c_char_p, i, ip, ip, C.POINTER(ll), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]
    L.tf_read_dense_mtx.argtypes = [C.c_char_p, ip, ip, C.POINTER(vp)]
    L.tf_lattice_preview.argtypes = [C.POINTER(Csr), i, i, i, ip, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), ip]
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != TF_OK:
        raise TileFusionError(rc, lib().tf_last_error().decode())


def np_ptr(a: np.ndarray) -> int:
    return a.ctypes.data
