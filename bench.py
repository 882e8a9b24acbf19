#!/usr/bin/env python
"""Benchmark of the fused sparse-dense chains on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c5|c3|c4] [--impl ours|reference]
                    [--mode stream|unfused] [--quick] [--dims X,Y,Z]

A step is one pass of the fused chain over one resident batch of synthetic input.  The headline workload
is the SpMM-SpMM chain D = A*(A*C) on the 3-D 7-point Laplacian of a 128^3 grid with 128 dense columns
(the one configuration on which the reference's CPU executor runs the identical full problem); with N
ranks every rank owns one 128^3 slab of a 128 x 128 x (128*N) grid (weak scaling) and exchanges one plane
of A*C with each neighbour per step.  After the headline the same process measures the GeMM-SpMM chain
D = A*(B*C) -- the 256^3 case split over the N ranks (strong scaling) and, on one GPU, the 256^2 case --
and reports them under "also".  One JSON line is printed by rank 0.
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

UNIT = "GFLOP/s"
METRICS = {"spmm_spmm": "fused SpMM-SpMM D=A*(A*C) GFLOP/s", "gemm_spmm": "fused GeMM-SpMM D=A*(B*C) GFLOP/s",
           "gcn": "2-layer GCN forward (fused GeMM-SpMM per layer) GFLOP/s", "sddmm_spmm": "fused SDDMM-SpMM GFLOP/s"}

GRAPH_WORKLOADS = {
    "c3": dict(chain="gcn", n=2_449_029, degree=25,
               label="2-layer GCN forward, fused GeMM-SpMM per layer: R-MAT n=2,449,029 avg degree 25 symmetrised "
                     "+ self loops, X n x 100 N(0,1), W1 100->256, W2 256->47 Glorot, ReLU between"),
    "c4": dict(chain="sddmm_spmm", n=1 << 20, degree=32,
               label="SDDMM-SpMM fp32: R-MAT n=1,048,576 avg degree 32, Q,K n x 64, V n x 128 N(0,1/8)"),
}

WORKLOADS = {
    # name: chain, grid dims (per rank for the weak-scaling case, whole job for the strong-scaling one), dense widths
    "c2": dict(chain="spmm_spmm", dims=(128, 128, 128), n=128, scaling="weak",
               label="SpMM-SpMM fp32 D=A*(A*C), 3-D 7-pt Laplacian 128^3 per GPU, C n x 128 uniform[-1,1]"),
    "c1": dict(chain="gemm_spmm", dims=(256, 256), k=64, n=64, scaling="weak",
               label="GeMM-SpMM fp32 D=A*(B*C), 2-D 5-pt Laplacian 256^2, B n x 64, C 64 x 64"),
    "c5": dict(chain="gemm_spmm", dims=(256, 256, 256), k=256, n=256, scaling="strong",
               label="GeMM-SpMM fp32 D=A*(B*C), 3-D 7-pt Laplacian 256^3 (whole job), B n x 256, C 256 x 256"),
}

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel on the full workload, from
# the ncu capture summarised in profiles/lattice_march_kernel_spmm_spmm_laplacian3d.md
DRAM_TRAFFIC = {"c2": 1_201_267_000 + 1_042_153_000}

# TileM values (bytes of cache per tile) of the reference's own sweep, fusion/scripts/run_exp.sh mode 7, thinned
TILE_M_SWEEP = (60_000, 300_000, 1_250_000)
CPU_TRIALS = 7  # fusion/example/SpMM_SpMM_SP_Demo.cpp:47


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
            nv, h = self._nv, self._h
            if nv is None:
                return
            names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
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
        try:  # NVML is brought up here, not in the thread: its start-up takes longer than a short timed region
            import pynvml as nv
            nv.nvmlInit()
            self._nv, self._h = nv, nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self._h, nv.NVML_CLOCK_SM)
        except Exception as e:
            self._nv = self._h = None
            self.reasons.add(f"unavailable:{type(e).__name__}")
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
def cpu_reference(workload: str, steps: int, warmup: int, sweep: bool = True):
    """Times the reference's fused CPU executor the way its own experiments do: variable-tile schedules for a
    sweep of cache budgets (TileM), AVX2 and -- where the host has it -- AVX-512 kernels, CPU_TRIALS runs each,
    best configuration reported; then `steps` more runs of that configuration are returned as the timed steps."""
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
    engines = []
    if use_ref:
        engines.append(("avx2", Ref(), 1))
        if wl["chain"] == "spmm_spmm" and Ref.avx512_available():
            engines.append(("avx512", Ref(avx512=True), 2))
    else:
        engines.append(("port", Oracle(), 0))
    orc = Oracle()
    t0 = time.time()
    tile_ms = TILE_M_SWEEP if sweep else (1_250_000,)
    trials = CPU_TRIALS if sweep else 3
    if wl["chain"] == "spmm_spmm":
        n = wl["n"]
        c = synth.uniform(3, (m, n))
        flops = synth.flops_spmm_spmm(nnz, nnz, n)
        d, ac = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)
        scheds = {tm: orc.inspect_variable(2, a[0], a[1], threads, tm, n) for tm in tile_ms}

        def run(eng, variant, sched):
            d.fill(0); ac.fill(0)
            t = time.perf_counter()
            if use_ref:
                eng.spmm_spmm(a, a, c, sched, threads=threads, variant=variant, out=(d, ac))
            else:
                eng.spmm_spmm(a, a, c, sched)
            return time.perf_counter() - t
        name = "spmmCsrSpmmCsrFusedVectorized2_32SP / ..Avx512SP"
    else:
        k, n = wl["k"], wl["n"]
        b, w = synth.uniform(2, (m, k)), synth.uniform(3, (k, n))
        flops = synth.flops_gemm_spmm(m, nnz, k, n)
        d, tmp = np.zeros((m, n), np.float32), np.zeros((m, n), np.float32)
        scheds = {tm: orc.inspect_variable(3, a[0], a[1], threads, tm, k, n) for tm in tile_ms}

        def run(eng, variant, sched):
            d.fill(0)
            t = time.perf_counter()
            if use_ref:
                eng.gemm_spmm(a, b, w, sched, threads=threads, variant=1, out=(d, tmp))
            else:
                eng.gemm_spmm(a, b, w, sched)
            return time.perf_counter() - t
        name = "forwardForOneLayerFusedParallelSeparatedVectorizedSP"
    scheds = {tm: s for tm, s in scheds.items() if s is not None}
    setup_s = time.time() - t0
    best = None
    table = {}
    for ename, eng, variant in engines:
        for tm, sched in scheds.items():
            for _ in range(max(warmup, 1)):
                run(eng, variant, sched)
            ts = [run(eng, variant, sched) for _ in range(trials)]
            table[f"{ename}/TileM={tm}"] = round(1e3 * float(np.median(ts)), 3)
            if best is None or np.median(ts) < best[0]:
                best = (float(np.median(ts)), ename, eng, variant, tm, sched)
    _, ename, eng, variant, tm, sched = best
    times = [run(eng, variant, sched) for _ in range(steps)]
    return dict(flops=flops, times=times, cores=cores, threads=threads, kind="reference" if use_ref else "port",
                sample=f"{'x'.join(map(str, dims))} grid, n={m}, nnz={nnz}; {name} with variable-tile schedules; best of "
                       f"TileM {list(tile_ms)} x kernels {[e[0] for e in engines]} by median of {trials} "
                       f"runs = {ename}/TileM={tm}; schedules + inputs {setup_s:.1f} s untimed",
                sweep_ms=table, sgemm=getattr(eng, "sgemm", None))


def cpu_port_graph(workload: str, n_rows: int):
    """CPU figure for the graph workloads: the oracle's plain-C restatement on a bounded sample of the same
    generator (the reference has no executor for the composed chains)."""
    from oracle.bindings import Oracle
    orc = Oracle()
    wl = GRAPH_WORKLOADS[workload]
    n = min(n_rows, 200_000)
    t0 = time.time()
    if workload == "c3":
        g = synth.rmat_gcn(1, n, wl["degree"])
        x, w1, w2 = synth.normal(2, (n, 100)), synth.glorot(3, 256, 100), synth.glorot(4, 47, 256)
        nnz = len(g[1])
        flops = synth.flops_gemm_spmm(n, nnz, 100, 256) + synth.flops_gemm_spmm(n, nnz, 256, 47)
        run = lambda: orc.gcn2(g, x, w1, w2)  # noqa: E731
    else:
        g = synth.rmat_pattern(1, n, wl["degree"])
        q, k, v = synth.normal(2, (n, 64), 0.125), synth.normal(3, (n, 64), 0.125), synth.normal(4, (n, 128), 0.125)
        nnz = len(g[1])
        flops = synth.flops_sddmm_spmm(nnz, 64, 128)
        run = lambda: orc.sddmm_spmm(g, q, k, v)  # noqa: E731
    setup = time.time() - t0
    run()
    ts = []
    for _ in range(3):
        t = time.perf_counter(); run(); ts.append(time.perf_counter() - t)
    ms = 1e3 * float(np.median(ts))
    return {"value": flops / (ms * 1e-3) / 1e9, "unit": UNIT, "cores": 1, "kind": "port", "ms": ms,
            "sample": f"same generator at n={n} rows, nnz={nnz}; plain-C restatement, one thread; setup {setup:.1f} s untimed"}


def print_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    if args.workload in GRAPH_WORKLOADS:
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no CPU executor for the composed graph chains "
                          "(2-layer GCN, SDDMM-SpMM); see cpu_baseline (kind port) of the GPU arm"}))
        return 0
    r = cpu_reference(args.workload, args.steps, max(args.warmup, 1))
    ms = 1e3 * float(np.mean(r["times"]))
    val = r["flops"] / (ms * 1e-3) / 1e9
    wl = WORKLOADS[args.workload]
    line = {"impl": "reference", "metric": METRICS[wl["chain"]], "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
            "scaling": wl["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["label"], "host": "CPU only"},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"],
                             "sweep_ms": r["sweep_ms"]},
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
    n = wl["n"]
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    t0 = time.time()
    if args.workload == "c3":
        ap, ai, ax = synth.rmat_gcn(1, n, wl["degree"])
        A = api.CSRMatrix(n, n, ap, ai, ax)
        nnz = A.nnz
        host = [synth.normal(2, (n, 100)), synth.glorot(3, 256, 100), synth.glorot(4, 47, 256)]
        x, w1, w2 = (torch.from_numpy(h).to(dev) for h in host)
        plans = (api.Plan("gemm_spmm", A, k=100, n_cols=256), api.Plan("gemm_spmm", A, k=256, n_cols=47))
        h1 = torch.empty((n, 256), device=dev)
        out = torch.empty((n, 47), device=dev)

        def step():
            plans[0].gemm_spmm(x, w1, h1, w_transposed=True, relu=True)
            plans[1].gemm_spmm(h1, w2, out, w_transposed=True, relu=False)
        h1_host, out_host = np.empty((n, 256), np.float32), np.empty((n, 47), np.float32)

        def step_host():  # the two fused layers through the host-pointer call (README-level executor)
            plans[0].gemm_spmm_host(host[0], host[1], h1_host, w_transposed=True, relu=True)
            plans[1].gemm_spmm_host(h1_host, host[2], out_host, w_transposed=True, relu=False)
        h2d = 4 * (n * 100 + 100 * 256 + n * 256 + 256 * 47)
        d2h = 4 * (n * 256 + n * 47)
        flops = synth.flops_gemm_spmm(n, nnz, 100, 256) + synth.flops_gemm_spmm(n, nnz, 256, 47)
        nbytes = synth.bytes_gemm_spmm(n, nnz, 100, 256) + synth.bytes_gemm_spmm(n, nnz, 256, 47)
        gather = 4 * nnz * (256 + 47)   # bytes of intermediate rows the two SpMMs gather, one row per nonzero
        launches = 2
        plan = plans[0]
    else:
        ap, ai, ax = synth.rmat_pattern(1, n, wl["degree"])
        A = api.CSRMatrix(n, n, ap, ai, ax)
        nnz = A.nnz
        host = [synth.normal(2, (n, 64), 0.125), synth.normal(3, (n, 64), 0.125), synth.normal(4, (n, 128), 0.125)]
        q, kk, v = (torch.from_numpy(h).to(dev) for h in host)
        out = torch.empty((n, 128), device=dev)
        plan = api.Plan("sddmm_spmm", A, k=64, n_cols=128)

        def step():
            plan.sddmm_spmm(q, kk, v, out)
        out_host = np.empty((n, 128), np.float32)

        def step_host():
            plan.sddmm_spmm_host(host[0], host[1], host[2], out_host)
        h2d, d2h = 4 * n * (64 + 64 + 128), 4 * n * 128
        flops = synth.flops_sddmm_spmm(nnz, 64, 128)
        nbytes = synth.bytes_sddmm_spmm(n, nnz, 64, 128)
        gather = 4 * nnz * (64 + 128)   # a row of K and a row of V per nonzero
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
    step_host()
    t0 = time.perf_counter()
    for _ in range(2):
        step_host()
    e_ms = (time.perf_counter() - t0) * 1e3 / 2
    peak, peak_kind = measured_peak_gbs()
    achieved = nbytes / (ms * 1e-3) / 1e9
    line = {"metric": METRICS[wl["chain"]], "value": flops / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["label"], "rows": n, "nnz": nnz, "max_row_nnz": int(np.diff(ap).max()),
                       "setup_s": round(setup_s, 1), "l2": "operands exceed the 126 MB L2; no flush"},
            "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": f"of {peak_kind}", "algorithmic_bytes_per_launch": nbytes,
                         "kernel": "stream_kernel (persistent executor)", "kernel_ms": ms,
                         "gather_bytes_per_step": gather, "gather_gbs": gather / (ms * 1e-3) / 1e9,
                         "gather_note": "one dense row per nonzero through L2 -> SM; random rows, so the HBM figure does not bound "
                                        "this workload: read gather_gbs against the ~13 TB/s L2 -> SM row-gather rate of this GPU"},
            "cpu_baseline": cpu_port_graph(args.workload, n) if not args.quick else None,
            "e2e": {"value": flops / (e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "host_buffers": "pageable"},
            "gpu_launches": launches * args.steps}
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm: one Laplacian workload on this rank set
# ---------------------------------------------------------------------------------------------
def tf32_peak(torch, dev):
    """Dense TF32 throughput of this GPU: torch.matmul with TF32 allowed (library figure), TFLOP/s."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a, b = torch.randn((n, n), device=dev), torch.randn((n, n), device=dev)
        for _ in range(2):
            a @ b
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); a @ b; e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * n ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def check_columns(torch, dist, chain, a_rows, in0, in1, d, r0, n_rows, fi, world):
    """Two columns of this rank's rows of D against an fp64 product formed on the host with scipy (every rank's
    rows of the intermediate column are gathered first): the outputs of the timed path, boundary rows included.
    Returns the largest relative L2 difference over the ranks (tolerance of the parity tests: 1e-5)."""
    import scipy.sparse as sp
    m, n = d.shape
    cols = [0, n - 1]
    if chain == "spmm_spmm":
        c = in0[:, cols].double().cpu().numpy()
        F = sp.csr_matrix((a_rows[2].astype(np.float64), fi, a_rows[0]), shape=(m, in0.shape[0]))
        t_loc = torch.from_numpy(F @ c).to(d.device)
    else:
        t_loc = (in0 @ in1[:, cols]).double()          # fp32 GEMM (TF32 off), two columns
    if world > 1:
        parts = [torch.empty_like(t_loc) for _ in range(world)]    # equal slabs
        dist.all_gather(parts, t_loc.contiguous())
        t_full = torch.cat(parts).cpu().numpy()
    else:
        t_full = t_loc.cpu().numpy()
    A = sp.csr_matrix((a_rows[2].astype(np.float64), a_rows[1], a_rows[0]), shape=(m, n_rows))
    want = A @ t_full
    got = d[:, cols].double().cpu().numpy()
    rel = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-300))
    if world > 1:
        t = torch.tensor([rel], device=d.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rel = float(t.item())
    return {"columns": cols, "max_rel_l2_over_ranks": rel, "ok": bool(rel <= 1e-5),
            "how": "fp64 scipy product of the whole chain for these columns, every rank's rows"}


def run_lattice_workload(name, args, ctx, headline):
    """Measures one of c1 / c2 / c5 on the ranks of `ctx`; returns the JSON fields on rank 0, None elsewhere."""
    import torch
    from tile_fusion_b200 import _lib, api, distributed, partition
    world, rank, dev, dist = ctx["world"], ctx["rank"], ctx["dev"], ctx["dist"]
    wl = WORKLOADS[name]
    chain, n = wl["chain"], wl["n"]
    k = wl.get("k", 0)
    dims = [int(v) for v in args.dims.split(",")] if args.dims else list(wl["dims"])
    if len(dims) != len(wl["dims"]):
        raise SystemExit(f"--dims: workload {name} has a {len(wl['dims'])}-D grid")
    strong = wl["scaling"] == "strong"
    if not strong and world > 1:
        dims[-1] *= world  # weak scaling: the grid grows along its slowest axis
    dims = tuple(dims)
    n_rows = int(np.prod(dims))
    bounds = partition.row_bounds(None, n_rows, world)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    m = r1 - r0
    t_setup = time.time()
    a_rows = synth.laplacian_rows(dims, r0, r1)
    nnz_local = len(a_rows[1])
    st = torch.cuda.current_stream().cuda_stream
    mode = api.MODE_STREAM if args.mode == "stream" else api.MODE_UNFUSED

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
            plan = api.Plan("spmm_spmm", A, n_cols=n, mode=mode)
            step = lambda: plan.spmm_spmm(in0, d)  # noqa: E731
        else:
            plan = api.Plan("gemm_spmm", A, k=k, n_cols=n, mode=mode)
            step = lambda: plan.gemm_spmm(in0, in1, d)  # noqa: E731
        rc = None
    else:
        # one C call per step: partition, ncclSend / ncclRecv of the halo rows and the three phases inside the library
        rc = distributed.NativeRankChain(chain, rank, world, r0, r1, a_rows, n, k=k, dist=dist, device=dev,
                                         mode=mode)
        if chain == "spmm_spmm":
            assert (rc.info["c_first"], rc.info["c_rows"]) == (lo, hi - lo)
        plan = api.Plan.adopt(rc)
        step = lambda: rc.step(in0, in1, d)  # noqa: E731
    setup_s = time.time() - t_setup

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    steps = args.steps if headline else max(3, min(args.steps, 10))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    with ClockSampler(ctx["local"]) as clk:  # samples from the warm-up on: the timed region alone lasts a few tens of ms
        for _ in range(args.warmup):
            step()
        plan.status()
        sync_all()
        ev[0].record()
        for i in range(steps):
            step()
            ev[i + 1].record()
        sync_all()
        # the timed region of a sub-millisecond step lasts a few milliseconds: keep the same launches going (untimed)
        # until the sampler has seen the clocks under this load for a tenth of a second
        t_obs = time.perf_counter()
        extra = 0
        while headline and world == 1 and time.perf_counter() - t_obs < 0.1 and extra < 400:   # (one rank: no collective to keep in step)
            step()
            extra += 1
            if extra % 20 == 0:
                torch.cuda.synchronize()
        sync_all()
    plan.status()
    step_trace = None
    if rc is not None:
        rc.status()
        # one more step, traced: where each rank's step spends its time (ms from the step's start)
        rc.trace(True)
        sync_all()
        step()
        mine = rc.trace(False) or {}
        t = torch.tensor([mine.get(k, -1.0) for k in ("phase0_done", "exchange_done", "phase2_done", "phase1_done", "step_done")],
                         device=dev, dtype=torch.float32)
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        step_trace = {"columns": ["phase0_done", "exchange_done", "phase2_done", "phase1_done", "step_done"],
                      "ms_from_step_start_per_rank": [[round(float(v), 4) for v in p.tolist()] for p in parts]}
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
    launches_per_step = plan.info()["launches"] if world == 1 else (3 if rc.info["boundary_rows"] else 2)
    if dist is not None:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        tot = torch.tensor([float(flops_local), float(bytes_local)], device=dev, dtype=torch.float64)
        dist.all_reduce(tot)
        flops_job = float(tot[0])
    else:
        flops_job = float(flops_local)
    ms_per_step = total_ms / steps
    value = flops_job / (ms_per_step * 1e-3) / 1e9

    peak, peak_kind = measured_peak_gbs()
    kernel_ms = float(np.mean(per_step))          # this rank's launches, CUDA events on the launching stream
    achieved = bytes_local / (kernel_ms * 1e-3) / 1e9
    threads = plan.info()["threads"]
    kernel = {128: "lattice_march_kernel", 672: "tile_pipeline_kernel"}.get(threads, "stream_kernel")
    if chain == "gemm_spmm" and threads == 128:
        kernel = "tc_gemm_kernel (dense producer) + lattice_march_kernel"
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_source": f"of {peak_kind}", "algorithmic_bytes_per_launch": bytes_local,
                "kernel": kernel + (" (persistent fused executor)" if "+" not in kernel else " (two launches per step)"),
                "kernel_ms": kernel_ms,
                "kernel_ms_min": float(np.min(per_step))}
    if world == 1 and args.mode == "stream" and name in DRAM_TRAFFIC and kernel == "lattice_march_kernel" and not args.dims:
        roofline["traffic"] = DRAM_TRAFFIC[name]
    if chain == "gemm_spmm" and rank == 0:
        # the dense producer multiplies three TF32 products per fp32 product: its floor is a tensor-core time
        if "tf32_tflops" not in ctx:
            ctx["tf32_tflops"] = tf32_peak(torch, dev)
        tf32 = ctx["tf32_tflops"]
        t_hbm = bytes_local / (peak * 1e9) * 1e3
        t_tc = 3 * 2.0 * m * k * n / (tf32 * 1e12) * 1e3
        roofline.update({"tf32_tflops_measured": tf32, "tf32_source": "torch.matmul 8192^3 with TF32 allowed, best of 5",
                         "hbm_floor_ms": t_hbm, "tensor_floor_ms": t_tc, "bound": "tensor" if t_tc > t_hbm else "hbm",
                         "frac_of_max_floor": max(t_hbm, t_tc) / kernel_ms,
                         "note": "frac = algorithmic bytes / time / HBM peak; frac_of_max_floor = max(HBM time, 3xTF32 tensor "
                                 "time) / time"})

    # ---- end to end through the host-pointer call (copies inside the timed region) ----
    e2e = None
    if world == 1 and (headline or not args.quick):
        e_steps = 5 if headline else 2

        def host_call(pinned):
            mk = (lambda s: torch.empty(s, pin_memory=True)) if pinned else (lambda s: torch.from_numpy(np.empty(s, np.float32)))
            if chain == "spmm_spmm":
                hin = [mk((m, n))]
                hin[0].copy_(in0[:m] if in0.shape[0] != m else in0)
                hout = mk((m, n))
                call = lambda: plan.spmm_spmm_host(hin[0].numpy(), hout.numpy())  # noqa: E731
            else:
                hin = [mk((m, k)), mk((k, n))]
                hin[0].copy_(in0); hin[1].copy_(in1)
                hout = mk((m, n))
                call = lambda: plan.gemm_spmm_host(hin[0].numpy(), hin[1].numpy(), hout.numpy())  # noqa: E731
            call()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(e_steps):
                call()
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) * 1e3 / e_steps, hin, hout
        # the extra workloads hand over pageable arrays only (pinning tens of GB takes longer than the run)
        e_ms, hin, hout = host_call(headline)
        same = bool(torch.equal(hout.to(dev), d))
        h2d = int(sum(t.numel() * 4 for t in hin))
        d2h = int(hout.numel() * 4)
        # what the link alone allows: the same bytes as two plain copies, one direction at a time
        scratch = torch.empty_like(d)
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(); in0[:hin[0].shape[0]].copy_(hin[0], non_blocking=True); e1.record()
        hout.copy_(scratch, non_blocking=True); e2.record()
        torch.cuda.synchronize()
        up_ms, down_ms = e0.elapsed_time(e1), e1.elapsed_time(e2)
        # ... and both directions at once (two streams): the floor of a pipelined call
        side = torch.cuda.Stream()
        d0, d1, d2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        side.wait_stream(torch.cuda.current_stream())
        d0.record()
        with torch.cuda.stream(side):
            hout.copy_(scratch, non_blocking=True)
            d2.record(side)
        in0[:hin[0].shape[0]].copy_(hin[0], non_blocking=True); d1.record()
        torch.cuda.synchronize()
        duplex_ms = max(d0.elapsed_time(d1), d0.elapsed_time(d2))
        e2e = {"value": flops_job / (e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e_ms, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": e_steps, "matches_device_path": same,
               "host_buffers": "pinned" if headline else "pageable",
               "link": {"h2d_only_ms": up_ms, "d2h_only_ms": down_ms, "h2d_gbs": hin[0].numel() * 4 / up_ms / 1e6,
                        "d2h_gbs": d2h / down_ms / 1e6, "both_directions_at_once_ms": duplex_ms}}
        del hin, hout, scratch
        if headline:  # the reference's call sites hand over plain new[] arrays (SpMM_SpMM_Demo_Utils.h:43-60)
            p_ms, _, _ = host_call(False)
            e2e["pageable"] = {"value": flops_job / (p_ms * 1e-3) / 1e9, "ms_per_step": p_ms}
    elif world > 1 and headline:
        # Every rank brings its rows from pinned host memory, runs the step and takes its rows of D back: the copies
        # of a rank are not overlapped with its step (the library's pipelined host-pointer call is single-GPU), the
        # ranks run side by side, each over its own PCIe link.
        e_steps = 3
        h_in = [torch.empty(t.shape, pin_memory=True) for t in ((in0,) if in1 is None else (in0, in1))]
        for h, t in zip(h_in, (in0, in1)):
            h.copy_(t)
        h_out = torch.empty(d.shape, pin_memory=True)

        def host_step():
            in0.copy_(h_in[0], non_blocking=True)
            if in1 is not None:
                in1.copy_(h_in[1], non_blocking=True)
            step()
            h_out.copy_(d, non_blocking=True)
        host_step()
        sync_all()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            host_step()
        sync_all()
        e_ms = (time.perf_counter() - t0) * 1e3 / e_steps
        t = torch.tensor([e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms = float(t.item())
        h2d = int(sum(h.numel() * 4 for h in h_in))
        e2e = {"value": flops_job / (e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e_ms, "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": int(h_out.numel() * 4) * world, "steps": e_steps, "host_buffers": "pinned",
               "matches_device_path": bool(torch.equal(h_out.to(dev), d)),
               "how": "per rank: upload of its rows, the device step, download of its rows of D, not overlapped; "
                      "max over ranks; bytes summed over ranks"}
        del h_in, h_out
    elif world > 1:
        e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
               "note": "measured for the headline workload only at N > 1 (pinning tens of GB per rank takes longer than the run)"}

    cpu = None
    if rank == 0 and world == 1 and not args.quick:
        r = cpu_reference(name, 3, 1, sweep=headline)
        # best configuration of the sweep, or its re-run if that came out faster
        cpu_ms = min(1e3 * float(np.median(r["times"])), min(r["sweep_ms"].values()))
        cpu = {"value": r["flops"] / (cpu_ms * 1e-3) / 1e9, "unit": UNIT, "cores": r["cores"], "kind": r["kind"],
               "sample": r["sample"], "ms": cpu_ms, "sweep_ms": r["sweep_ms"], "sgemm": r["sgemm"]}

    parity = check_columns(torch, dist, chain, a_rows, in0, in1, d, r0, n_rows, fi if chain == "spmm_spmm" else None, world)

    info, tiles = plan.info(), plan.tile_info()
    if rc is not None:
        rc.close()
    else:
        plan.close()
    del d, in0, in1
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"metric": METRICS[chain], "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": wl["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["label"] + (" -- grid overridden by --dims (a profiling case)" if args.dims else ""),
                       "grid": "x".join(map(str, dims)), "rows": n_rows,
                       "rows_per_gpu": m, "mode": args.mode, "ring_rows": info["ring_rows"], "grid_ctas": info["grid"],
                       "threads_per_cta": threads, "tiles": tiles, "setup_s": round(setup_s, 1),
                       "l2": "inputs (>= 1 GB per step) exceed the 126 MB L2; no flush" if bytes_local > 5e8 else
                             "operands (tens of MB) fit the 126 MB L2 and are not flushed between steps: a warm-L2 figure",
                       "partition": f"row blocks over {world} GPU(s), halo rows of the intermediate over NCCL",
                       "parity": parity, **({"step_trace": step_trace} if step_trace else {})},
            "clocks": clk.summary(), "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(launches_per_step * steps)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(GRAPH_WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="stream", choices=["stream", "unfused"])
    ap.add_argument("--quick", action="store_true", help="kernel timing only: no CPU baseline, no 'also' workloads")
    ap.add_argument("--dims", default="", help="grid of a lattice workload, e.g. 128,128,32: a small case of the same kernel "
                                               "for profiler captures (the line then names that grid, not the workload's)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return print_reference(args)
    if args.workload in GRAPH_WORKLOADS:
        if args.gpus != 1:
            print(json.dumps({"impl": args.impl, "unavailable": "graph workloads c3/c4 run on one GPU"}))
            return 0
        return run_graph_workload(args)

    import torch
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
    ctx = dict(world=world, rank=rank, local=local, dev=dev, dist=dist)

    line = run_lattice_workload(args.workload, args, ctx, headline=True)
    also = []
    if args.workload == "c2" and not args.quick:
        # the reference's headline chain: GeMM-SpMM, 256^3 over these ranks (strong scaling), 256^2 on one GPU
        for extra in (["c5", "c1"] if world == 1 else ["c5"]):
            try:
                r = run_lattice_workload(extra, args, ctx, headline=False)
            except Exception as e:  # keep the headline line
                r = {"config": {"workload": WORKLOADS[extra]["label"]}, "error": f"{type(e).__name__}: {e}"}
            if rank == 0 and r is not None:
                also.append(r)
    if rank == 0:
        line["also"] = also
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
