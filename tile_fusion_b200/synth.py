"""Seeded synthetic inputs for the fused sparse-dense chains.

The reference draws its dense operands from an unseeded ``std::random_device``
(fusion/src/Fusion_Utils.cpp:301-311) or fills them with ones
(fusion/example/SpMM_SpMM_Demo_Utils.h:57-59) and reads its sparse operands from
SuiteSparse / OGB files that are not shipped.  This module defines reproducible
stand-ins with the same shapes: a counter-based generator (any slice can be
produced independently, on the host here or on the device by the library's
``tf_fill_*`` kernels, with identical bits), grid Laplacians in natural order
and R-MAT graphs.  All sparse matrices are CSR, int32 indices, sorted columns.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def unit(seed: int, start: int, count: int) -> np.ndarray:
    """u(seed, idx) in [0, 1) for idx = start .. start+count-1 (float64, 24 significant bits)."""
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64)
        z = _splitmix64(np.uint64(seed) * _GOLDEN + idx)
    return (z >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)


def uniform(seed: int, shape, start: int = 0, chunk: int = 1 << 24) -> np.ndarray:
    """float32 uniform[-1, 1): 2*u - 1 (exact in fp32: u has 24 bits)."""
    count = int(np.prod(shape))
    out = np.empty(count, dtype=np.float32)
    for s in range(0, count, chunk):
        n = min(chunk, count - s)
        out[s:s + n] = (2.0 * unit(seed, start + s, n) - 1.0).astype(np.float32)
    return out.reshape(shape)


def normal(seed: int, shape, sigma: float = 1.0, start: int = 0, chunk: int = 1 << 23) -> np.ndarray:
    """float32 N(0, sigma^2) by Box-Muller on (u(2i), u(2i+1)), evaluated in float32."""
    count = int(np.prod(shape))
    out = np.empty(count, dtype=np.float32)
    for s in range(0, count, chunk):
        n = min(chunk, count - s)
        u = unit(seed, 2 * (start + s), 2 * n)
        u1 = (1.0 - u[0::2]).astype(np.float32)  # (0, 1]
        u2 = u[1::2].astype(np.float32)
        r = np.sqrt(np.float32(-2.0) * np.log(u1))
        out[s:s + n] = np.float32(sigma) * r * np.cos(np.float32(2.0 * np.pi) * u2)
    return out.reshape(shape)


def glorot(seed: int, fan_out: int, fan_in: int) -> np.ndarray:
    """Glorot-uniform weight stored [fan_out, fan_in] as the reference's torch layers do
    (binding-project/gcn-e2e-training/FusedGCNLayer.py:10-11)."""
    lim = np.float32(np.sqrt(6.0 / (fan_in + fan_out)))
    return uniform(seed, (fan_out, fan_in)) * lim


def laplacian(dims, dtype=np.float32):
    """Grid Laplacian in natural (x fastest) order: diagonal 2*len(dims), off-diagonals -1.

    dims = (nx,), (nx, ny) or (nx, ny, nz).  Returns (Ap, Ai, Ax) with sorted columns.
    """
    dims = tuple(int(d) for d in dims)
    n = int(np.prod(dims))
    idx = np.arange(n, dtype=np.int64)
    strides, coords, s = [], [], 1
    for d in dims:
        strides.append(s)
        coords.append((idx // s) % d)
        s *= d
    # candidate neighbours in ascending column order: -s_k (k descending), 0, +s_k (k ascending)
    cols, valid, vals = [], [], []
    for k in reversed(range(len(dims))):
        cols.append(idx - strides[k]); valid.append(coords[k] > 0); vals.append(-1.0)
    cols.append(idx); valid.append(np.ones(n, dtype=bool)); vals.append(2.0 * len(dims))
    for k in range(len(dims)):
        cols.append(idx + strides[k]); valid.append(coords[k] < dims[k] - 1); vals.append(-1.0)
    valid = np.stack(valid, axis=1)
    cols = np.stack(cols, axis=1)
    vals = np.broadcast_to(np.asarray(vals, dtype=dtype), valid.shape)
    ap = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(valid.sum(axis=1), out=ap[1:])
    assert ap[-1] < 2 ** 31
    return ap.astype(np.int32), cols[valid].astype(np.int32), np.ascontiguousarray(vals[valid])


def rmat_edges(seed: int, n: int, n_edges: int, a=0.57, b=0.19, c=0.19, chunk: int = 1 << 22):
    """R-MAT edge list (src, dst) with ids >= n rejected; scale = ceil(log2 n)."""
    scale = max(1, int(np.ceil(np.log2(n))))
    src_l, dst_l, have, ctr = [], [], 0, 0
    while have < n_edges:
        m = min(chunk, max(1024, int((n_edges - have) * 1.3) + 16))
        src = np.zeros(m, dtype=np.int64)
        dst = np.zeros(m, dtype=np.int64)
        for bit in range(scale):
            u = unit(seed, ctr, m); ctr += m
            right = (u >= a) & (u < a + b) | (u >= a + b + c)      # quadrants b, d -> column bit
            down = u >= a + b                                      # quadrants c, d -> row bit
            src = (src << 1) | down
            dst = (dst << 1) | right
        ok = (src < n) & (dst < n)
        src_l.append(src[ok]); dst_l.append(dst[ok]); have += int(ok.sum())
    return np.concatenate(src_l)[:n_edges], np.concatenate(dst_l)[:n_edges]


def _csr_from_pairs(n, src, dst):
    key = np.unique(src.astype(np.int64) * n + dst.astype(np.int64))
    rows = key // n
    ai = (key % n).astype(np.int32)
    ap = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=n), out=ap[1:])
    assert ap[-1] < 2 ** 31
    return ap.astype(np.int32), ai


def rmat_gcn(seed: int, n: int, avg_degree: int = 25):
    """Symmetrised R-MAT graph with self loops, values 1/sqrt(deg_i*deg_j) where deg = row nnz
    including the self loop (fusion/gcn/SingleLayer/GCN_Single_Layer_SP_Demo_Utils.h:40-53)."""
    src, dst = rmat_edges(seed, n, (avg_degree * n) // 2)
    loops = np.arange(n, dtype=np.int64)
    ap, ai = _csr_from_pairs(n, np.concatenate([src, dst, loops]), np.concatenate([dst, src, loops]))
    deg = np.diff(ap).astype(np.float64)
    rows = np.repeat(np.arange(n), np.diff(ap))
    ax = (1.0 / np.sqrt(deg[rows] * deg[ai])).astype(np.float32)
    return ap, ai, ax


def rmat_pattern(seed: int, n: int, avg_degree: int = 32):
    """Directed R-MAT sparsity pattern (deduplicated), values 1 -- the attention mask of the
    SDDMM-SpMM chain.  Rows left empty by the generator get their diagonal entry."""
    src, dst = rmat_edges(seed, n, avg_degree * n)
    loops = np.arange(n, dtype=np.int64)
    ap0, _ = _csr_from_pairs(n, src, dst)
    empty = loops[np.diff(ap0) == 0]
    ap, ai = _csr_from_pairs(n, np.concatenate([src, empty]), np.concatenate([dst, empty]))
    return ap, ai, np.ones(ai.shape[0], dtype=np.float32)


# ---------------------------------------------------------------------------
# FLOP / byte counts (algorithmic: every input once, output once, A once, the
# intermediate never)
# ---------------------------------------------------------------------------
def flops_gemm_spmm(n, nnz, k, ncols):
    return 2 * n * k * ncols + 2 * nnz * ncols


def flops_spmm_spmm(nnz_a, nnz_b, ncols):
    return 2 * (nnz_a + nnz_b) * ncols


def flops_sddmm_spmm(nnz, kq, nv):
    return 2 * nnz * kq + nnz + 2 * nnz * nv


def bytes_gemm_spmm(n, nnz, k, ncols):
    return 4 * (n * k + k * ncols + n * ncols + 2 * nnz + (n + 1))


def bytes_spmm_spmm(n, nnz, ncols):
    return 4 * (2 * n * ncols + 2 * nnz + (n + 1))


def bytes_sddmm_spmm(n, nnz, kq, nv):
    return 4 * (2 * n * kq + 2 * n * nv + 2 * nnz + (n + 1))


def laplacian_rows(dims, row0: int, row1: int, dtype=np.float32):
    """Rows [row0, row1) of laplacian(dims) with GLOBAL column ids (what one rank of a row-block
    partition owns).  Returns (Ap, Ai, Ax) with Ap starting at 0."""
    dims = tuple(int(d) for d in dims)
    idx = np.arange(row0, row1, dtype=np.int64)
    strides, coords, s = [], [], 1
    for d in dims:
        strides.append(s)
        coords.append((idx // s) % d)
        s *= d
    cols, valid, vals = [], [], []
    for k in reversed(range(len(dims))):
        cols.append(idx - strides[k]); valid.append(coords[k] > 0); vals.append(-1.0)
    cols.append(idx); valid.append(np.ones(len(idx), dtype=bool)); vals.append(2.0 * len(dims))
    for k in range(len(dims)):
        cols.append(idx + strides[k]); valid.append(coords[k] < dims[k] - 1); vals.append(-1.0)
    valid = np.stack(valid, axis=1)
    cols = np.stack(cols, axis=1)
    vals = np.broadcast_to(np.asarray(vals, dtype=dtype), valid.shape)
    ap = np.zeros(len(idx) + 1, dtype=np.int64)
    np.cumsum(valid.sum(axis=1), out=ap[1:])
    return ap.astype(np.int32), cols[valid].astype(np.int64), np.ascontiguousarray(vals[valid])
