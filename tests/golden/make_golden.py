"""Generates tests/golden/*.npz by running the UNMODIFIED reference (compiled in place into
oracle/_ref/libtf_ref.so by `make -C oracle ref`) on seeded inputs.

Run where the reference tree is mounted:   python tests/golden/make_golden.py
The fixtures hold only what the reference produced (schedule arrays, statistics, outputs) and the
parameters of each case; inputs are regenerated from their seeds by tile_fusion_b200.synth.
"""
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
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    print("wrote", len(manifest), "fixtures")


if __name__ == "__main__":
    main()
