#!/usr/bin/env python
"""Benchmark of the fused sparse-dense chains on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c5] [--impl ours|reference]

A step is one pass of the fused chain over one resident batch of synthetic input.  The default
workload is the SpMM-SpMM chain D = A*(A*C) on the 3-D 7-point Laplacian of a 128^3 grid with
128 dense columns; with N ranks every rank owns one 128^3 slab of a 128 x 128 x (128*N) grid
(weak scaling) and exchanges one plane of A*C with each neighbour per step.  One JSON line is
printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tile_fusion_b200 import synth  # noqa: E402

METRIC = "fused D=A*(B*C) GFLOP/s"
UNIT = "GFLOP/s"

GRAPH_WORKLOADS = {
    "c3": dict(label="2-layer GCN forward, fused GeMM-SpMM per layer: R-MAT n=2,449,029 avg degree 25 symmetrised "
                     "+ self loops, X n x 100 N(0,1), W1 100->256, W2 256->47 Glorot, ReLU between",
               n=2_449_029, degree=25),
    "c4": dict(label="SDDMM-SpMM fp32: R-MAT n=1,048,576 avg degree 32, Q,K n x 64, V n x 128 N(0,1/8)",
               n=1 << 20, degree=32),
}

WORKLOADS = {
    # name: (chain, grid dims per rank (x, y, z-per-rank), dense widths)
    "c2": dict(chain="spmm_spmm", dims=(128, 128, 128), n=128,
               label="SpMM-SpMM fp32 D=A*(A*C), 3-D 7-pt Laplacian 128^3 per GPU, C n x 128 uniform[-1,1]"),
    "c1": dict(chain="gemm_spmm", dims=(256, 256), k=64, n=64,
               label="GeMM-SpMM fp32 D=A*(B*C), 2-D 5-pt Laplacian 256^2, B n x 64, C 64 x 64"),
    "c5": dict(chain="gemm_spmm", dims=(256, 256, 256), k=256, n=256,
               label="GeMM-SpMM fp32 D=A*(B*C), 3-D 7-pt Laplacian 256^3 (whole job), B n x 256, C 256 x 256"),
}


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (captured on a quarter-size case and scaled by rows)
DRAM_TRAFFIC = {"c2": 4 * (713_756_416 + 496_346_368)}


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only NVML)."""

    def __init__(self, index: int, period=0.005):
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None

    def _loop(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown if hasattr(nv, "nvmlClocksEventReasonHwSlowdown") else 0x8,
                     "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
            while not self._stop.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
                time.sleep(self.period)
        except Exception as e:  # keep the bench alive without clock data
            self.reasons.add(f"unavailable:{type(e).__name__}")

    def __enter__(self):
        self._thr = threading.Thread(target=self._loop, daemon=True)
        self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thr.join(timeout=2)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU executor (oracle/_ref, compiled in place), all host cores
# ---------------------------------------------------------------------------------------------
def cpu_reference(workload: str, steps: int, warmup: int):
    from oracle.bindings import Oracle, Ref
    wl = WORKLOADS[workload]
    cores = os.cpu_count() or 1
    threads = cores
    dims = wl["dims"]
    # bounded sample: the full single-GPU workload where it fits the host in seconds, else a slab
    if workload == "c5":
        dims = (256, 256, 32)
    a = synth.laplacian(dims)
    m, nnz = len(a[0]) - 1, len(a[1])
    use_ref = Ref.available()
    eng = Ref() if use_ref else Oracle()
    orc = Oracle()
    t0 = time.time()
    if wl["chain"] == "spmm_spmm":
        n = wl["n"]
        sched = orc.inspect_variable(2, a[0], a[1], threads, 1_250_000, n)
        c = synth.uniform(3, (m, n))
        flops = synth.flops_spmm_spmm(nnz, nnz, n)
        d, ac = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)

        def run():
            d.fill(0); ac.fill(0)
            t = time.perf_counter()
            if use_ref:
                eng.spmm_spmm(a, a, c, sched, threads=threads, variant=1, out=(d, ac))
            else:
                eng.spmm_spmm(a, a, c, sched)
            return time.perf_counter() - t
        name = "spmmCsrSpmmCsrFusedVectorized2_32SP + variable-tile schedule (cache 1.25 MB)"
    else:
        k, n = wl["k"], wl["n"]
        sched = orc.inspect_variable(3, a[0], a[1], threads, 1_250_000, k, n)
        b, w = synth.uniform(2, (m, k)), synth.uniform(3, (k, n))
        flops = synth.flops_gemm_spmm(m, nnz, k, n)
        d, tmp = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)

        def run():
            d.fill(0)
            t = time.perf_counter()
            if use_ref:
                eng.gemm_spmm(a, b, w, sched, threads=threads, variant=1, out=(d, tmp))
            else:
                eng.gemm_spmm(a, b, w, sched)
            return time.perf_counter() - t
        name = "forwardForOneLayerFusedParallelSeparatedVectorizedSP + variable-tile schedule (cache 1.25 MB)"
    setup_s = time.time() - t0
    for _ in range(warmup):
        run()
    times = [run() for _ in range(steps)]
    return dict(flops=flops, times=times, cores=cores, threads=threads, kind="reference" if use_ref else "port",
                sample=f"{'x'.join(map(str, dims))} grid, n={m}, nnz={nnz}; {name}; setup+inspector {setup_s:.1f} s untimed",
                sgemm=getattr(eng, "sgemm", None))


def print_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    r = cpu_reference(args.workload, args.steps, max(args.warmup, 1))
    ms = 1e3 * float(np.mean(r["times"]))
    val = r["flops"] / (ms * 1e-3) / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[args.workload]["label"], "host": "CPU only"},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# graph workloads (single GPU): 2-layer GCN and SDDMM-SpMM on R-MAT graphs
# ---------------------------------------------------------------------------------------------
def run_graph_workload(args):
    import torch
    from tile_fusion_b200 import api
    wl = GRAPH_WORKLOADS[args.workload]
    n = wl["n"] if not args.dims else int(args.dims)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    t0 = time.time()
    if args.workload == "c3":
        ap, ai, ax = synth.rmat_gcn(1, n, wl["degree"])
        A = api.CSRMatrix(n, n, ap, ai, ax)
        nnz = A.nnz
        x = torch.from_numpy(synth.normal(2, (n, 100))).to(dev)
        w1 = torch.from_numpy(synth.glorot(3, 256, 100)).to(dev)
        w2 = torch.from_numpy(synth.glorot(4, 47, 256)).to(dev)
        plans = (api.Plan("gemm_spmm", A, k=100, n_cols=256), api.Plan("gemm_spmm", A, k=256, n_cols=47))
        h1 = torch.empty((n, 256), device=dev)
        out = torch.empty((n, 47), device=dev)

        def step():
            plans[0].gemm_spmm(x, w1, h1, w_transposed=True, relu=True)
            plans[1].gemm_spmm(h1, w2, out, w_transposed=True, relu=False)
        flops = synth.flops_gemm_spmm(n, nnz, 100, 256) + synth.flops_gemm_spmm(n, nnz, 256, 47)
        nbytes = synth.bytes_gemm_spmm(n, nnz, 100, 256) + synth.bytes_gemm_spmm(n, nnz, 256, 47)
        launches = 2
        plan = plans[0]
    else:
        ap, ai, ax = synth.rmat_pattern(1, n, wl["degree"])
        A = api.CSRMatrix(n, n, ap, ai, ax)
        nnz = A.nnz
        q = torch.from_numpy(synth.normal(2, (n, 64), 0.125)).to(dev)
        kk = torch.from_numpy(synth.normal(3, (n, 64), 0.125)).to(dev)
        v = torch.from_numpy(synth.normal(4, (n, 128), 0.125)).to(dev)
        out = torch.empty((n, 128), device=dev)
        plan = api.Plan("sddmm_spmm", A, k=64, n_cols=128)

        def step():
            plan.sddmm_spmm(q, kk, v, out)
        flops = synth.flops_sddmm_spmm(nnz, 64, 128)
        nbytes = synth.bytes_sddmm_spmm(n, nnz, 64, 128)
        launches = 1
    setup_s = time.time() - t0
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(0) as clk:
        for _ in range(args.warmup):
            step()
        plan.status()
        torch.cuda.synchronize()
        ev[0].record()
        for i in range(args.steps):
            step()
            ev[i + 1].record()
        torch.cuda.synchronize()
    plan.status()
    ms = ev[0].elapsed_time(ev[-1]) / args.steps
    peak, peak_kind = measured_peak_gbs()
    achieved = nbytes / (ms * 1e-3) / 1e9
    line = {"metric": METRIC, "value": flops / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["label"], "rows": n, "nnz": nnz, "max_row_nnz": int(np.diff(ap).max()),
                       "setup_s": round(setup_s, 1), "l2": "operands exceed the 126 MB L2; no flush"},
            "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": f"of {peak_kind}", "algorithmic_bytes_per_launch": nbytes,
                         "kernel": "stream_kernel (persistent executor)", "kernel_ms": ms},
            "cpu_baseline": None, "e2e": None, "gpu_launches": launches * args.steps}
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(GRAPH_WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="stream", choices=["stream", "unfused"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--rows-per-block", type=int, default=0)
    ap.add_argument("--slack", type=int, default=-1)
    ap.add_argument("--ring-mb", type=int, default=0)
    ap.add_argument("--ctas-per-sm", type=int, default=0)
    ap.add_argument("--tile-slots", type=int, default=0)
    ap.add_argument("--tile-max-bz", type=int, default=0)
    ap.add_argument("--tile-double", type=int, default=0)
    ap.add_argument("--tile-pipeline", type=int, default=0, help="<0: run gather tiles on the two-CTA kernel")
    ap.add_argument("--dims", default="", help="override the per-rank grid, e.g. 128,128,32 (profiling on a small case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload in GRAPH_WORKLOADS:
        if args.impl == "reference" or args.gpus != 1:
            print(json.dumps({"impl": args.impl, "unavailable": "graph workloads c3/c4 run on one GPU, our arm only"}))
            return 0
        return run_graph_workload(args)
    if args.impl == "reference":
        return print_reference(args)

    import torch
    from tile_fusion_b200 import _lib, api, distributed, partition

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    wl = WORKLOADS[args.workload]
    chain, n = wl["chain"], wl["n"]
    k = wl.get("k", 0)
    dims = list(wl["dims"]) if not args.dims else [int(x) for x in args.dims.split(",")]
    strong = args.workload == "c5"
    if not strong and world > 1:
        dims[-1] *= world  # weak scaling: the grid grows along its slowest axis
    dims = tuple(dims)
    n_rows = int(np.prod(dims))
    bounds = partition.row_bounds(None, n_rows, world)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    m = r1 - r0
    a_rows = synth.laplacian_rows(dims, r0, r1)
    nnz_local = len(a_rows[1])
    st = torch.cuda.current_stream().cuda_stream
    mode = api.MODE_STREAM if args.mode == "stream" else api.MODE_UNFUSED
    plan_kw = dict(rows_per_block=args.rows_per_block, slack_blocks=args.slack, ctas_per_sm=args.ctas_per_sm,
                   tile_slots=args.tile_slots, tile_max_bz=args.tile_max_bz, tile_double_buffer=args.tile_double, tile_pipeline=args.tile_pipeline,
                   ring_bytes=args.ring_mb << 20 if args.ring_mb > 0 else (0 if args.ring_mb == 0 else -1))

    def fill(t, seed, offset):
        _lib.check(_lib.lib().tf_fill_uniform(t.data_ptr(), t.numel(), seed, offset, st))

    # ---- operands resident on the device ----
    if chain == "spmm_spmm":
        ids, fi = partition.compact_columns(a_rows[1])          # own rows of C plus ghost rows
        lo, hi = int(ids[0]), int(ids[-1]) + 1
        assert hi - lo == len(ids)                               # a contiguous extended slab
        c_ext = torch.empty((hi - lo, n), device=dev)
        fill(c_ext, 3, lo * n)
        in0, in1 = c_ext, None
        flops_local = synth.flops_spmm_spmm(nnz_local, nnz_local, n)
        bytes_local = synth.bytes_spmm_spmm(m, nnz_local, n)
    else:
        b = torch.empty((m, k), device=dev)
        fill(b, 2, r0 * k)
        w = torch.empty((k, n), device=dev)
        fill(w, 3, 0)
        in0, in1 = b, w
        flops_local = synth.flops_gemm_spmm(m, nnz_local, k, n)
        bytes_local = synth.bytes_gemm_spmm(m, nnz_local, k, n)
    d = torch.empty((m, n), device=dev)

    if world == 1:
        A = api.CSRMatrix(m, m, a_rows[0], a_rows[1].astype(np.int32), a_rows[2])
        if chain == "spmm_spmm":
            plan = api.Plan("spmm_spmm", A, n_cols=n, mode=mode, **plan_kw)
            step = lambda: plan.spmm_spmm(in0, d)  # noqa: E731
        else:
            plan = api.Plan("gemm_spmm", A, k=k, n_cols=n, mode=mode, **plan_kw)
            step = lambda: plan.gemm_spmm(in0, in1, d)  # noqa: E731
        rc = None
    else:
        mine = partition.halo_of(a_rows[1], r0, r1)
        halos = [None] * world
        dist.all_gather_object(halos, mine)
        lay = partition.make_layout(rank, bounds, halos)
        if chain == "spmm_spmm":
            rc = distributed.RankChain("spmm_spmm", lay, a_rows, n, first_rows=(a_rows[0], fi, a_rows[2], len(ids)),
                                       device=dev, rows_per_block=args.rows_per_block)
        else:
            rc = distributed.RankChain("gemm_spmm", lay, a_rows, n, k=k, device=dev, rows_per_block=args.rows_per_block)
        plan = rc.plan
        step = lambda: rc.step(in0, in1, d, dist=dist)  # noqa: E731

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local) as clk:  # samples from the warm-up on: the timed region alone lasts a few tens of ms
        for _ in range(args.warmup):
            step()
        plan.status()
        sync_all()
        ev[0].record()
        for i in range(args.steps):
            step()
            ev[i + 1].record()
        sync_all()
    plan.status()
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    launches_per_step = plan.info()["launches"] if world == 1 else (3 if len(rc.lay.boundary_rows) else 2)
    if dist is not None:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        tot = torch.tensor([float(flops_local), float(bytes_local)], device=dev, dtype=torch.float64)
        dist.all_reduce(tot)
        flops_job, bytes_job = float(tot[0]), float(tot[1])
    else:
        flops_job, bytes_job = float(flops_local), float(bytes_local)
    ms_per_step = total_ms / args.steps
    value = flops_job / (ms_per_step * 1e-3) / 1e9

    peak, peak_kind = measured_peak_gbs()
    kernel_ms = float(np.mean(per_step))          # this rank's launches, CUDA events on the launching stream
    achieved = bytes_local / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_source": f"of {peak_kind}", "algorithmic_bytes_per_launch": bytes_local,
                "kernel": {128: "lattice_march_kernel", 672: "tile_pipeline_kernel"}.get(plan.info()["threads"], "stream_kernel")
                          + " (persistent fused executor)", "kernel_ms": kernel_ms,
                "kernel_ms_min": float(np.min(per_step))}
    if world == 1 and not args.dims and args.mode == "stream" and args.workload in DRAM_TRAFFIC:
        roofline["traffic"] = DRAM_TRAFFIC[args.workload]

    # ---- end to end through the host-pointer call (pinned host buffers, copies inside) ----
    e2e = None
    if not args.no_e2e and world == 1:
        e_steps = max(3, min(args.steps, 5))
        if chain == "spmm_spmm":
            hin = [torch.empty((m, n), pin_memory=True)]
            hin[0].copy_(in0)
            hout = torch.empty((m, n), pin_memory=True)
            call = lambda: plan.spmm_spmm_host(hin[0].numpy(), hout.numpy())  # noqa: E731
        else:
            hin = [torch.empty((m, k), pin_memory=True), torch.empty((k, n), pin_memory=True)]
            hin[0].copy_(in0); hin[1].copy_(in1)
            hout = torch.empty((m, n), pin_memory=True)
            call = lambda: plan.gemm_spmm_host(hin[0].numpy(), hin[1].numpy(), hout.numpy())  # noqa: E731
        call()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            call()
        torch.cuda.synchronize()
        e_ms = (time.perf_counter() - t0) * 1e3 / e_steps
        same = bool(torch.equal(hout.to(dev), d))
        e2e = {"value": flops_job / (e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e_ms,
               "h2d_bytes_per_step": int(sum(t.numel() * 4 for t in hin)), "d2h_bytes_per_step": int(hout.numel() * 4),
               "steps": e_steps, "matches_device_path": same}
    elif world > 1:
        e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
               "note": "the host-pointer call is single-GPU; measured at --gpus 1"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        r = cpu_reference(args.workload, 3, 1)
        cpu_ms = 1e3 * float(np.median(r["times"]))
        cpu = {"value": r["flops"] / (cpu_ms * 1e-3) / 1e9, "unit": UNIT, "cores": r["cores"], "kind": r["kind"],
               "sample": r["sample"], "ms": cpu_ms, "sgemm": r["sgemm"]}

    if rank == 0:
        info = plan.info()
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": wl["label"], "grid": "x".join(map(str, dims)), "rows": n_rows,
                           "rows_per_gpu": m, "mode": args.mode, "ring_rows": info["ring_rows"], "grid_ctas": info["grid"],
                           "items": info["items"], "tiles": plan.tile_info(), "l2": "inputs (>= 1 GB per step) exceed the 126 MB L2; no flush",
                           "partition": f"row blocks over {world} GPU(s), halo rows of the intermediate over NCCL"},
                "clocks": clk.summary(), "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": int(launches_per_step * args.steps)}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
