"""Sweep driver: the fused chains over a list of matrix files, one CSV line per (matrix, chain, width).

    python -m tile_fusion_b200.sweep --folder DIR --list LIST.txt [--chain spmm_spmm|gemm_spmm] [--bcols 32,64,128]
                                     [--k 64] [--trials 7] [--out results.csv] [--check]

Stands in for the reference's experiment scripts (fusion/scripts/run_exp.sh: for every matrix of a list
file under a folder and every dense width, run the demo binary and append its CSV line) and for the matrix
ingestion of its demo mains (get_matrix_from_parameter, fusion/src/Fusion_Utils.cpp:252-272: *.mtx and
*.smtx files).  The SuiteSparse / DLMC / OGB collections the reference sweeps are not shipped with it; any
directory of such files works.  Columns: matrix, rows, cols, nnz, chain, b_cols, k, executor (threads per
CTA of the kernel the plan chose), tiles, plan_s (analysis time, reported separately as the reference
does), ms_median, ms_min, gflops, check (max relative difference to the unfused executor, with --check).
"""
from __future__ import annotations

import argparse
import csv
import os
import sys
import time

import numpy as np


def run_one(path, chain, n_cols, k, trials, check):
    import torch

    from . import api, synth
    A = api.read_matrix(path)
    if A.M != A.N:
        raise ValueError("the chains need a square matrix")
    dev = torch.device("cuda", torch.cuda.current_device())
    t0 = time.perf_counter()
    if chain == "spmm_spmm":
        plan = api.Plan("spmm_spmm", A, n_cols=n_cols)
        ins = [torch.from_numpy(synth.uniform(3, (A.M, n_cols))).to(dev)]
        flops = synth.flops_spmm_spmm(A.nnz, A.nnz, n_cols)
        call = lambda p, d: p.spmm_spmm(ins[0], d)  # noqa: E731
    else:
        plan = api.Plan("gemm_spmm", A, k=k, n_cols=n_cols)
        ins = [torch.from_numpy(synth.uniform(2, (A.M, k))).to(dev), torch.from_numpy(synth.uniform(3, (k, n_cols))).to(dev)]
        flops = synth.flops_gemm_spmm(A.M, A.nnz, k, n_cols)
        call = lambda p, d: p.gemm_spmm(ins[0], ins[1], d)  # noqa: E731
    plan_s = time.perf_counter() - t0
    d = torch.empty((A.M, n_cols), device=dev)
    for _ in range(2):
        call(plan, d)
    plan.status()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(trials + 1)]
    ev[0].record()
    for i in range(trials):
        call(plan, d)
        ev[i + 1].record()
    torch.cuda.synchronize()
    plan.status()
    ts = [ev[i].elapsed_time(ev[i + 1]) for i in range(trials)]
    err = ""
    if check:
        kw = dict(mode=api.MODE_UNFUSED, tile_slots=-1, tensor_cores=-1)
        ref = api.Plan(chain, A, n_cols=n_cols, lattice_march=-1, **kw) if chain == "spmm_spmm" else \
            api.Plan(chain, A, k=k, n_cols=n_cols, **kw)
        d0 = torch.empty_like(d)
        call(ref, d0)
        ref.status()
        den = float(d0.abs().max()) or 1.0
        err = f"{float((d - d0).abs().max()) / den:.3e}"
        ref.close()
    info, tiles = plan.info(), plan.tile_info()
    plan.close()
    ms = float(np.median(ts))
    return [os.path.basename(str(path)), A.M, A.N, A.nnz, chain, n_cols, k if chain == "gemm_spmm" else "", info["threads"],
            tiles["consumer"][3], f"{plan_s:.3f}", f"{ms:.4f}", f"{min(ts):.4f}", f"{flops / (ms * 1e-3) / 1e9:.1f}", err]


HEADER = ["matrix", "rows", "cols", "nnz", "chain", "b_cols", "k", "executor_threads", "tiles", "plan_s", "ms_median", "ms_min",
          "gflops", "check"]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--folder", default=".")
    ap.add_argument("--list", help="text file with one matrix file name per line (default: every *.mtx / *.smtx of the folder)")
    ap.add_argument("--chain", default="spmm_spmm", choices=["spmm_spmm", "gemm_spmm"])
    ap.add_argument("--bcols", default="32,64,128")
    ap.add_argument("--k", type=int, default=64)
    ap.add_argument("--trials", type=int, default=7)
    ap.add_argument("--out", default="-")
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    if args.list:
        with open(args.list) as f:
            names = [ln.strip() for ln in f if ln.strip() and not ln.startswith("#")]
    else:
        names = sorted(n for n in os.listdir(args.folder) if n.endswith((".mtx", ".smtx")))
    out = sys.stdout if args.out == "-" else open(args.out, "w", newline="")
    w = csv.writer(out)
    w.writerow(HEADER)
    failed = 0
    for name in names:
        for bc in (int(x) for x in args.bcols.split(",")):
            try:
                w.writerow(run_one(os.path.join(args.folder, name), args.chain, bc, args.k, args.trials, args.check))
            except Exception as e:  # one bad file does not end the sweep
                failed += 1
                w.writerow([name, "", "", "", args.chain, bc, "", "", "", "", "", "", "", f"error: {type(e).__name__}: {e}"])
            out.flush()
    if out is not sys.stdout:
        out.close()
    return 1 if failed and failed == len(names) * len(args.bcols.split(",")) else 0


if __name__ == "__main__":
    sys.exit(main())
