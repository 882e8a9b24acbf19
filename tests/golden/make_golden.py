"""Generates tests/golden/*.npz by running the UNMODIFIED reference (compiled in place into
oracle/_ref/libtf_ref.so by `make -C oracle ref`) on seeded inputs.

Run where the reference tree is mounted:   python tests/golden/make_golden.py
The fixtures hold only what the reference produced (schedule arrays, statistics, outputs) and the
parameters of each case; inputs are regenerated from their seeds by tile_fusion_b200.synth.

Besides the compiled C++ reference, two more pieces of the reference are run here:
  * sddmm_cpu (codegen/triton/sddmm.py:173-184, a numba function).  The module cannot be imported as a whole --
    its top level reads dataset lists from its author's home directory -- so the function definition alone is
    taken out of the file's syntax tree and compiled, unchanged, with numba.
  * GnnTensorSpInputs::normalizeAdjacencyMatrix (fusion/gcn/SingleLayer/GCN_Single_Layer_SP_Demo_Utils.h:40-53),
    through oracle/_ref (see oracle/Makefile).
"""
import ast
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.bindings import Ref, build  # noqa: E402
from tile_fusion_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def matrix(spec):
    kind = spec[0]
    if kind == "lap":
        return synth.laplacian(spec[1])
    if kind == "rmat_gcn":
        return synth.rmat_gcn(spec[1], spec[2], spec[3])
    raise ValueError(kind)


# (name, matrix spec, inspector kind, params)
SCHEDULE_CASES = [
    ("lap1d_1000_fixed", ("lap", (1000,)), 1, dict(threads=4, iter_per_part=64)),
    ("lap1d_1000_vt_spmm", ("lap", (1000,)), 2, dict(threads=4, tile_m=20000, bcol=32)),
    ("lap2d_64_fixed_ip64", ("lap", (64, 64)), 1, dict(threads=4, iter_per_part=64)),
    ("lap2d_64_fixed_ip512", ("lap", (64, 64)), 1, dict(threads=2, iter_per_part=512)),
    ("lap2d_64_vt_gemm", ("lap", (64, 64)), 3, dict(threads=4, tile_m=300000, bcol=64, ccol=64)),
    ("lap2d_64_vt_gemm_small", ("lap", (64, 64)), 3, dict(threads=4, tile_m=60000, bcol=32, ccol=32)),
    ("lap2d_64_vt_spmm", ("lap", (64, 64)), 2, dict(threads=4, tile_m=60000, bcol=64)),
    ("lap2d_64_vt_spmm_threads", ("lap", (64, 64)), 4, dict(threads=4, tile_m=60000, bcol=64)),
    ("lap3d_16_vt_spmm", ("lap", (16, 16, 16)), 2, dict(threads=2, tile_m=100000, bcol=32)),
    ("lap3d_16_vt_gemm", ("lap", (16, 16, 16)), 3, dict(threads=2, tile_m=100000, bcol=32, ccol=32)),
    ("rmat_2048_fixed", ("rmat_gcn", 11, 2048, 8), 1, dict(threads=4, iter_per_part=128)),
    ("rmat_2048_vt_spmm", ("rmat_gcn", 11, 2048, 8), 2, dict(threads=4, tile_m=40000, bcol=32)),
    ("rmat_2048_vt_gemm", ("rmat_gcn", 11, 2048, 8), 3, dict(threads=4, tile_m=80000, bcol=32, ccol=32)),
    ("rmat_2048_vt_spmm_threads", ("rmat_gcn", 11, 2048, 8), 4, dict(threads=4, tile_m=40000, bcol=32)),
]

# (name, matrix spec, chain, dense widths, schedule case parameters)
OUTPUT_CASES = [
    ("out_spmm_spmm_lap2d_24", ("lap", (24, 24)), "spmm_spmm", dict(n=32),
     2, dict(threads=2, tile_m=30000, bcol=32)),
    ("out_spmm_spmm_rmat_512", ("rmat_gcn", 5, 512, 6), "spmm_spmm", dict(n=32),
     1, dict(threads=2, iter_per_part=64)),
    ("out_gemm_spmm_lap2d_24", ("lap", (24, 24)), "gemm_spmm", dict(k=16, n=32),
     3, dict(threads=2, tile_m=20000, bcol=16, ccol=32)),
    ("out_gemm_spmm_rmat_512", ("rmat_gcn", 5, 512, 6), "gemm_spmm", dict(k=24, n=64),
     1, dict(threads=2, iter_per_part=64)),
]


# (name, pattern spec, Kq): S = A .* (Q K^T) by the reference's sddmm_cpu; Q, K ~ N(0, 1/8) seeds 2, 3
SDDMM_CASES = [
    ("sddmm_rmat_1024_k32", ("rmat_pattern", 7, 1024, 8), 32),
    ("sddmm_rmat_1500_k64", ("rmat_pattern", 9, 1500, 6), 64),
]

# (name, graph spec): values of D^-1/2 (A + I) D^-1/2 by the reference's normalizeAdjacencyMatrix from all-ones values
NORMALIZE_CASES = [("gcn_norm_rmat_1500", ("rmat_gcn", 5, 1500, 8))]

# 3-D Laplacian outputs at N = 128: every 4th row of D is kept, plus sums over the whole of D
OUTPUT3D_CASES = [
    ("out3d_spmm_spmm_lap_16", ("lap", (16, 16, 16)), "spmm_spmm", dict(n=128), 2, dict(threads=2, tile_m=200000, bcol=128)),
    ("out3d_gemm_spmm_lap_16", ("lap", (16, 16, 16)), "gemm_spmm", dict(k=64, n=128), 3,
     dict(threads=2, tile_m=400000, bcol=64, ccol=128)),
]


def reference_sddmm_cpu(ref_root):
    """The reference's own sddmm_cpu, compiled from its definition in codegen/triton/sddmm.py."""
    import numba
    from numba import njit
    path = os.path.join(ref_root, "codegen", "triton", "sddmm.py")
    with open(path) as f:
        src = f.read()
    node = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "sddmm_cpu")
    ns = {"np": np, "numba": numba, "njit": njit}
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
    return ns["sddmm_cpu"]


def main():
    build(ref=True)
    ref = Ref(use_mkl_sgemm=False)  # plain-loop sgemm: fixtures do not depend on an MKL build
    manifest = {}
    for name, spec, kind, prm in SCHEDULE_CASES:
        ap, ai, ax = matrix(spec)
        s = ref.inspect(kind, ap, ai, prm["threads"], iter_per_part=prm.get("iter_per_part", 1),
                        tile_m=prm.get("tile_m", 1), bcol=prm.get("bcol", 1), ccol=prm.get("ccol", 1))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), n1=s.n1, ptr1=s.ptr1, ptr2=s.ptr2, id=s.id,
                            type=s.type, ker=s.ker_begin if s.ker_begin is not None else np.zeros(0, np.int32),
                            has_ker=s.ker_begin is not None, stats=s.stats[:5])
        manifest[name] = dict(matrix=list(spec), kind=kind, params=prm)
    for name, spec, chain, dims, kind, prm in OUTPUT_CASES:
        a = matrix(spec)
        m = len(a[0]) - 1
        s = ref.inspect(kind, a[0], a[1], prm["threads"], iter_per_part=prm.get("iter_per_part", 1),
                        tile_m=prm.get("tile_m", 1), bcol=prm.get("bcol", 1), ccol=prm.get("ccol", 1))
        if chain == "spmm_spmm":
            c = synth.uniform(3, (m, dims["n"]))
            d, _ = ref.spmm_spmm(a, a, c, s, threads=2, variant=1)
            d_unfused = ref.spmm(a[0], a[1], a[2], ref.spmm(a[0], a[1], a[2], c, threads=2), threads=2)
        else:
            b = synth.uniform(2, (m, dims["k"]))
            w = synth.uniform(3, (dims["k"], dims["n"]))
            d, _ = ref.gemm_spmm(a, b, w, s, threads=2, variant=1)
            d_unfused = ref.gemm_spmm_unfused(a, b, w, threads=2)
        assert np.array_equal(d, d_unfused), name  # the reference's own self-check (fused == unfused)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), D=d)
        manifest[name] = dict(matrix=list(spec), chain=chain, dims=dims, kind=kind, params=prm)
    ref_root = os.environ.get("TF_REFERENCE_ROOT", "/root/reference")
    sddmm_cpu = reference_sddmm_cpu(ref_root)
    for name, spec, kq in SDDMM_CASES:
        ap, ai, ax = synth.rmat_pattern(spec[1], spec[2], spec[3])
        n = len(ap) - 1
        q, k = synth.normal(2, (n, kq), 0.125), synth.normal(3, (n, kq), 0.125)
        s_val = sddmm_cpu(ap.astype(np.int32), ai.astype(np.int32), ax.astype(np.float32), q, k, n, n, kq)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), S=s_val)
        manifest[name] = dict(matrix=list(spec), kq=kq)
    for name, spec in NORMALIZE_CASES:
        ap, ai, _ = synth.rmat_gcn(spec[1], spec[2], spec[3])
        x = ref.normalize_adjacency(ap, ai, np.ones(len(ai)))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), Ax=x.astype(np.float32))
        manifest[name] = dict(matrix=list(spec))
    for name, spec, chain, dims, kind, prm in OUTPUT3D_CASES:
        a = matrix(spec)
        m = len(a[0]) - 1
        s = ref.inspect(kind, a[0], a[1], prm["threads"], tile_m=prm["tile_m"], bcol=prm["bcol"], ccol=prm.get("ccol", 1))
        if chain == "spmm_spmm":
            d, _ = ref.spmm_spmm(a, a, synth.uniform(3, (m, dims["n"])), s, threads=2, variant=1)
        else:
            d, _ = ref.gemm_spmm(a, synth.uniform(2, (m, dims["k"])), synth.uniform(3, (dims["k"], dims["n"])), s,
                                 threads=2, variant=1)
        rows = np.arange(0, m, 4)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), rows=rows, D=d[rows],
                            total=np.float64(d.astype(np.float64).sum()), sq=np.float64((d.astype(np.float64) ** 2).sum()))
        manifest[name] = dict(matrix=list(spec), chain=chain, dims=dims, kind=kind, params=prm)
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    print("wrote", len(manifest), "fixtures")


if __name__ == "__main__":
    main()
