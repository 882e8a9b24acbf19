"""The reference's torch operator library ``sw_gcn`` on CUDA tensors.

Importing this module registers, under the same names and with the same argument order as
``binding-project/main.cpp:133-142`` of the reference::

    torch.ops.sw_gcn.inspect(adj, m_tile_size)                                   -> [level_ptr, mix_ptr, partition]
    torch.ops.sw_gcn.inspect_vt_ro(adj, in_dim, out_dim, cache_size, threads)    -> [level_ptr, mix_ptr, l2_ptr]
    torch.ops.sw_gcn.fusedGeMMSpMM(adj, feature, weight, schedule, threads)      -> adj @ (feature @ weight.T)
    torch.ops.sw_gcn.fusedGeMMSpMM_vt_ro(adj, feature, weight, schedule, threads, max_tile_size)
    torch.ops.sw_gcn.geMMSpMM_f_bw(adj, feature, weight, schedule, threads)
    torch.ops.sw_gcn.unfused_gcn_forward(adj, feature, weight, threads)
    torch.ops.sw_gcn.cachedSpMMGeMM(af, weight, threads)                          -> af @ weight.T

``adj`` is a torch sparse-CSR tensor (int32 indices, fp32 values), ``weight`` is stored ``[out, in]`` as the
reference's layers do (``gcn-e2e-training/FusedGCNLayer.py:10-11``), everything lives on the GPU and the results
take part in autograd: the backward is the reference's (``src/Functions.cpp:819-1043``, ``:1192-1244``),
``dX = (A dY) W`` and ``dW = (A dY)^T X`` -- like the reference it multiplies by ``A``, not ``A^T``, i.e. it
assumes the symmetric adjacency of a GCN.  The forward runs the library's fused GeMM-SpMM executor; the sparse
product of the backward runs the library's CSR SpMM, its two dense products are plain library GEMMs.

The schedule tensors have the reference's layout (level pointers, per-partition kernel boundaries, row ids) and
come from the library's inspector for the same cache budget; the GPU executor plans its own tiles and does not
read them back (they are accepted and ignored), so a layer written for the reference
(``FusedGCNLayer.forward``: ``forward_fn(adj, x, weight, schedule, num_threads, max_tile_size)``) runs unchanged.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib, api

_LIB = torch.library.Library("sw_gcn", "DEF")
_plans: dict = {}


def _csr_of(adj: torch.Tensor):
    """(key, CSRMatrix on the host, device arrays) of a sparse-CSR adjacency; cached per tensor storage."""
    if adj.layout != torch.sparse_csr:
        raise ValueError("sw_gcn: the adjacency must be a torch sparse CSR tensor")
    crow, col, val = adj.crow_indices(), adj.col_indices(), adj.values()
    key = (crow.data_ptr(), col.data_ptr(), val.data_ptr(), adj.shape[0], int(val.numel()), val._version)
    hit = _plans.get(("csr", key))
    if hit is None:
        A = api.CSRMatrix(adj.shape[0], adj.shape[1], crow.to(torch.int32).cpu().numpy(), col.to(torch.int32).cpu().numpy(),
                          val.to(torch.float32).cpu().numpy())
        dev = (crow.to(torch.int32).cuda().contiguous(), col.to(torch.int32).cuda().contiguous(),
               val.to(torch.float32).cuda().contiguous())
        if len(_plans) > 64:
            for p in list(_plans.values()):
                if isinstance(p, api.Plan):
                    p.close()
            _plans.clear()
        hit = _plans[("csr", key)] = (A, dev)
    return key, hit[0], hit[1]


def _plan(adj, k, n, unfused=False):
    key, A, _ = _csr_of(adj)
    pk = ("plan", key, k, n, unfused)
    p = _plans.get(pk)
    if p is None:
        p = _plans[pk] = api.Plan("gemm_spmm", A, k=k, n_cols=n, mode=api.MODE_UNFUSED if unfused else api.MODE_STREAM)
    return p


def _spmm(adj, x):
    """A @ x with the library's CSR SpMM."""
    _, _, (ap, ai, ax) = _csr_of(adj)
    x = x.contiguous().float()
    out = torch.empty((adj.shape[0], x.shape[1]), device=x.device, dtype=torch.float32)
    _lib.check(_lib.lib().tf_spmm_dev(ap.data_ptr(), ai.data_ptr(), ax.data_ptr(), adj.shape[0], x.data_ptr(), x.shape[1],
                                      out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out


class _FusedGeMMSpMM(torch.autograd.Function):
    """Forward D = A (X W^T) on the fused executor; backward as FusedGeMMSpMMROAdj::backward
    (binding-project/src/Functions.cpp:1192-1244)."""

    @staticmethod
    def forward(ctx, adj, feature, weight, unfused):
        x = feature.contiguous().float()
        w = weight.contiguous().float()
        out = torch.empty((adj.shape[0], w.shape[0]), device=x.device, dtype=torch.float32)
        _plan(adj, x.shape[1], w.shape[0], unfused).gemm_spmm(x, w, out, w_transposed=True)
        ctx.adj = adj
        ctx.save_for_backward(x, w)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, w = ctx.saved_tensors
        ag = _spmm(ctx.adj, grad_out)                      # A dY (the reference multiplies by A: symmetric adjacency)
        grad_x = ag @ w if ctx.needs_input_grad[1] else None
        grad_w = ag.t() @ x if ctx.needs_input_grad[2] else None
        return None, grad_x, grad_w, None


class _CachedSpMMGeMM(torch.autograd.Function):
    """ForwardCachingAF (binding-project/src/Functions.cpp): out = AF W^T for a first layer whose A X is cached."""

    @staticmethod
    def forward(ctx, af, weight):
        ctx.save_for_backward(af, weight)
        return af @ weight.t()

    @staticmethod
    def backward(ctx, grad_out):
        af, weight = ctx.saved_tensors
        return (grad_out @ weight if ctx.needs_input_grad[0] else None), grad_out.t() @ af


def _schedule_tensors(adj, kind, **prm):
    _, A, _ = _csr_of(adj)
    s = api.inspector(A, prm.pop("threads"), kind=kind, **prm)
    level = torch.from_numpy(np.concatenate([s.ptr1, np.zeros(max(0, 3 - len(s.ptr1)), np.int32)])[:3].astype(np.int32))
    mix = torch.from_numpy(np.concatenate([np.zeros(2, np.int32), s.ker_begin]).astype(np.int32)) if s.ker_begin is not None \
        else torch.zeros(2, dtype=torch.int32)
    ids = torch.from_numpy(s.id[s.type == 1].astype(np.int32)) if len(s.id) else torch.zeros(0, dtype=torch.int32)
    return [level, mix, ids]


def _inspect(adj, m_tile_size):
    """Fixed tiles of m_tile_size rows (createSchedule, binding-project/src/Functions.cpp:551-627)."""
    return _schedule_tensors(adj, api.INSPECT_FIXED, threads=1, iter_per_partition=max(1, int(m_tile_size)))


def _inspect_vt(adj, in_dim, out_dim, cache_size, num_threads):
    """Variable tiles under a cache budget (inspect_vt, binding-project/main.cpp:51-88)."""
    return _schedule_tensors(adj, api.INSPECT_VT_GEMM, threads=max(1, int(num_threads)), tile_m=int(cache_size),
                             b_cols=int(in_dim), c_cols=int(out_dim))


_LIB.define("inspect(Tensor adj, int m_tile_size) -> Tensor[]")
_LIB.define("inspect_vt_ro(Tensor adj, int in_dim, int out_dim, int cache_size, int num_threads) -> Tensor[]")
_LIB.define("fusedGeMMSpMM(Tensor adj, Tensor feature, Tensor weight, Tensor[] schedule, int num_threads) -> Tensor")
_LIB.define("fusedGeMMSpMM_vt_ro(Tensor adj, Tensor feature, Tensor weight, Tensor[] schedule, int num_threads, "
            "int max_tile_size) -> Tensor")
_LIB.define("geMMSpMM_f_bw(Tensor adj, Tensor feature, Tensor weight, Tensor[] schedule, int num_threads) -> Tensor")
_LIB.define("unfused_gcn_forward(Tensor adj, Tensor feature, Tensor weight, int num_threads) -> Tensor")
_LIB.define("cachedSpMMGeMM(Tensor af, Tensor weight, int num_threads) -> Tensor")

# CompositeImplicitAutograd: the implementations call autograd Functions themselves, as the reference's ops do.
_LIB.impl("inspect", _inspect, "CompositeImplicitAutograd")
_LIB.impl("inspect_vt_ro", _inspect_vt, "CompositeImplicitAutograd")
_LIB.impl("fusedGeMMSpMM", lambda adj, f, w, sched, nt: _FusedGeMMSpMM.apply(adj, f, w, False), "CompositeImplicitAutograd")
_LIB.impl("fusedGeMMSpMM_vt_ro", lambda adj, f, w, sched, nt, mts: _FusedGeMMSpMM.apply(adj, f, w, False),
          "CompositeImplicitAutograd")
_LIB.impl("geMMSpMM_f_bw", lambda adj, f, w, sched, nt: _FusedGeMMSpMM.apply(adj, f, w, False), "CompositeImplicitAutograd")
_LIB.impl("unfused_gcn_forward", lambda adj, f, w, nt: _FusedGeMMSpMM.apply(adj, f, w, True), "CompositeImplicitAutograd")
_LIB.impl("cachedSpMMGeMM", lambda af, w, nt: _CachedSpMMGeMM.apply(af, w), "CompositeImplicitAutograd")
