#!/usr/bin/env python
"""Benchmark of the Shfl-BW hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Workload (config.workload): the headline SpMM -- M = N = K = 4096, V = 64, density 0.1,
row permutation on, seeded mask (seed 2021), fp16 uniform[-1,1) values and dense operand,
fp32 accumulation, fp16 output.  One step = one SpMM launch over one 4096-column batch of
the dense operand.  Several batches (B, D buffer pairs, > L2 in aggregate) are rotated so
every step reads its dense operand from HBM.  With N GPUs every rank runs the same workload
on its own batches (weak scaling; the sparse operand is replicated, no collective on the
data path); time is the max over ranks.

Printed JSON (one line, rank 0):
  value      nonzero-only TFLOP/s (2 * nnz * N / t), inputs resident in HBM
  dense_equivalent_tflops   2*M*K*N / t (what the reference's tool prints as "effective")
  roofline   achieved algorithmic GB/s of the SpMM kernel against the measured HBM peak
  e2e        same metric through the host-buffer C-ABI call (H2D + kernel + D2H per step)
  cpu_baseline  the reference's CPU check timed on this box on a column slice
  spconv     the headline SpConv (16x14x14x512 -> 2048, 3x3) measured the same way
  reference_gpu_kernel  the reference's own CUDA kernels (sm_100a build) on the same inputs

--impl reference times the reference's CPU implementation (oracle/_ref) on all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_ = K_ = N_ = 4096
V_ = 64
DENSITY = 0.1
SEED = 2021
CONV = dict(B=16, H=14, W=14, C=512, F=2048, R=3, S=3, stride=1)
METRIC = "spmm_nonzero_tflops"
UNIT = "TFLOP/s"

# DRAM bytes (read + write) of one SpMM kernel launch on the workload above, from the ncu
# capture summarised in profiles/panel_umma_spmm_4096_v64.md (37.1 MB read + 4.6 MB written;
# the D tile stays in L2 past the end of the launch).
NCU_DRAM_BYTES_PER_LAUNCH = 41_759_104


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), tflops=float(d["bf16_tflops"]),
                    tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def spmm_bytes(nnzb, V, X, M, K_touched, N, permuted=True):
    """Compulsory bytes of one SpMM: values + indices + indptr + permutation + B once + D once."""
    return 2 * nnzb * V + 4 * nnzb + 4 * (X + 1) + (4 * M if permuted else 0) + 2 * K_touched * N + 2 * M * N


class ClockSampler:
    """nvidia-smi sampling in a child process (read-only queries) while the timed region runs."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime as dt
        rows, inside = [], []
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) != 8:
                continue
            try:
                ts = dt.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                row = (ts, float(parts[1]), float(parts[2]), parts[4:8])
            except ValueError:
                continue
            rows.append(row)
            if t0 <= ts <= t1:
                inside.append(row)
        use, window = (inside, "timed region") if inside else (rows, "warm-up + timed region")
        if not use:
            return None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in use for n, v in zip(names, r[3]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[1] for r in use), "sm_max_mhz": use[0][2], "reasons": reasons,
                "samples": len(use), "window": window}


def capture_steps(torch, launch, steps, stream, use_graph=True):
    """Capture G consecutive steps (G = largest divisor of `steps` up to 200) into a CUDA graph.
    Returns (run, G): run() executes exactly `steps` steps on `stream`; G == 0 means plain launches.
    launch(i, raw_stream) enqueues step i."""
    G = max((g for g in range(1, min(steps, 200) + 1) if steps % g == 0), default=0) if use_graph else 0
    if G < 2:
        return (lambda: [launch(i, stream.cuda_stream) for i in range(steps)]), 0
    side = torch.cuda.Stream()
    side.wait_stream(stream)
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            cap = torch.cuda.current_stream().cuda_stream
            for i in range(G):
                launch(i, cap)
    torch.cuda.synchronize()
    graph.replay()                          # one untimed replay (graph upload)
    torch.cuda.synchronize()
    return (lambda: [graph.replay() for _ in range(steps // G)]), G


def build_problem(sb):
    m = sb.BlockwiseSpMatrix().init_random(M_, K_, V_, 1, DENSITY, True, SEED, values="uniform")
    return m


def run_ours(args):
    import torch
    import shflbw_sparse_nn_b200 as sb
    from shflbw_sparse_nn_b200.build import build_library

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build_library()
    if dist:
        dist.barrier()

    pk = peaks()
    m = build_problem(sb)
    m.transform_and_sync_device()
    nnzb, X = m.nnzb, M_ // V_
    nnz = nnzb * V_
    k_touched = int(np.unique(m.indices).size)
    flops_nz = 2.0 * nnz * N_
    flops_dense = 2.0 * M_ * K_ * N_
    bytes_alg = spmm_bytes(nnzb, V_, X, M_, k_touched, N_)

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.float16)

    NB = 4  # 4 x (33.5 MB B + 33.5 MB D) = 268 MB > 126 MB L2
    Bs = [dev(sb.uniform_half(100 + rank * 16 + i, K_ * N_).reshape(K_, N_)) for i in range(NB)]
    Ds = [torch.zeros((M_, N_), dtype=torch.float16, device="cuda") for _ in range(NB)]
    ops = [sb.SpmmBlockwiseOp().initialize(m, N_, Bs[i], Ds[i]) for i in range(NB)]
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream

    def step(i):
        ops[i % NB]._call_raw(sptr)

    # raw exec without Python-side wrapping overhead
    from shflbw_sparse_nn_b200 import _cabi
    import ctypes as C
    lib = _cabi.lib()
    for op in ops:
        st = C.byref(op._state)
        op._call_raw = (lambda st_: (lambda s: lib.shflbw_spmm_exec(st_, s)))(st)

    W = max(3, args.warmup)
    sampler = ClockSampler(local) if rank == 0 else None
    time.sleep(0.05)
    for i in range(W):
        step(i)
    torch.cuda.synchronize()

    # The timed loop is launch-gap sensitive (a ~41 us kernel per step): consecutive steps are
    # captured once into a CUDA graph and the graph is replayed.
    run_steps, G = capture_steps(torch, lambda i, raw: ops[i % NB]._call_raw(raw), args.steps, stream,
                                 use_graph=not args.no_graph)
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record(stream)
    run_steps()
    e1.record(stream)
    torch.cuda.synchronize()
    t_wall1 = time.time()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    ms_total = e0.elapsed_time(e1)
    if dist:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    m.device_status()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    ms_step = ms_total / args.steps
    value = world * flops_nz / (ms_step * 1e-3) / 1e12

    t_kernel = ms_step * 1e-3  # one kernel per step, launched back to back on one stream
    t_tc, t_hbm = flops_nz / (pk["tflops"] * 1e12), bytes_alg / (pk["hbm_gbs"] * 1e9)
    bound = "hbm" if t_hbm >= t_tc else "tensor"
    if bound == "hbm":
        achieved, peak, runit = bytes_alg / t_kernel / 1e9, pk["hbm_gbs"], "GB/s"
    else:
        achieved, peak, runit = flops_nz / t_kernel / 1e12, pk["tflops"], "TFLOP/s"
    roofline = {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": runit,
                "frac": round(achieved / peak, 4), "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                "peak_source": pk["source"], "algorithmic_bytes": bytes_alg, "algorithmic_flops": flops_nz,
                "kernel": "panel_umma_kernel<V=64,TM=2,KS=64,STAGES=5,PW=8,MODE=3>", "kernel_us": round(t_kernel * 1e6, 3),
                "t_roof_us": round(max(t_tc, t_hbm) * 1e6, 3)}

    out = {
        "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": W,
        "ms_per_step": round(ms_step, 6), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "SpMM M=N=K=4096 V=64 density=0.1 row-permute seed=2021 fp16 uniform[-1,1)",
                   "nnzb": nnzb, "batches_rotated": NB, "l2": "inputs larger than L2 (4 x 67 MB rotated)",
                   "per_gpu": "one 4096-column batch per step on every GPU; sparse operand replicated",
                   "launch": (f"CUDA graph of {G} steps replayed {args.steps // G}x" if G else "one host launch per step")},
        "dense_equivalent_tflops": round(world * flops_dense / (ms_step * 1e-3) / 1e12, 2),
        "roofline": roofline, "gpu_launches": args.steps * ops[0].launches_per_exec, "clocks": clocks,
    }

    if args.quick:
        if rank == 0 and world == 1:
            out["spconv"] = bench_spconv(sb, torch, pk, steps=30, warmup=5, use_graph=not args.no_graph)
        if dist:
            dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps(out))
        return

    # ---- end to end through the host-buffer C-ABI call (H2D + kernel + D2H inside the timing) ----
    e2e_steps = max(3, min(args.steps, 10))
    Bh = torch.from_numpy(sb.uniform_half(500 + rank, K_ * N_).reshape(K_, N_).view(np.int16)).pin_memory()
    Dh = torch.zeros((M_, N_), dtype=torch.int16).pin_memory()
    for _ in range(2):
        sb.spmm_host(m, N_, Bh, Dh)
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        sb.spmm_host(m, N_, Bh, Dh)   # synchronous: returns after the D2H copy completed
    t_e2e = (time.perf_counter() - t0) / e2e_steps
    if dist:
        t = torch.tensor([t_e2e], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_e2e = float(t.item())
    out["e2e"] = {"value": round(world * flops_nz / t_e2e / 1e12, 4), "unit": UNIT,
                  "h2d_bytes_per_step": 2 * K_ * N_, "d2h_bytes_per_step": 2 * M_ * N_,
                  "ms_per_step": round(t_e2e * 1e3, 4), "steps": e2e_steps,
                  "call": "shflbw_spmm_host (pinned host B and D)"}

    if rank == 0 and world == 1:
        out["spconv"] = bench_spconv(sb, torch, pk, use_graph=not args.no_graph)
        out["reference_gpu_kernel"] = bench_reference_gpu(sb, torch, m, Bs[0], Ds[0])
        out["cpu_baseline"] = cpu_baseline_sample(m, threads=1, budget_s=12.0)
        out["cpu_baseline"].pop("t_probe", None)
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out))


def bench_spconv(sb, torch, pk, steps=300, warmup=20, use_graph=True):
    c = CONV
    f = sb.BlockwiseSpFilter().init_random(c["F"], c["R"], c["S"], c["C"], V_, 1, DENSITY, True, SEED, values="uniform")
    f.transform_and_sync_device()
    NBc = 10  # 10 x (3.2 + 12.8 MB) = 160 MB > L2
    xs = [torch.from_numpy(sb.uniform_half(900 + i, c["B"] * c["H"] * c["W"] * c["C"]).view(np.int16)).cuda().view(torch.float16)
          for i in range(NBc)]
    os_ = [torch.zeros((c["B"], c["H"], c["W"], c["F"]), dtype=torch.float16, device="cuda") for _ in range(NBc)]
    ops = [sb.SpconvBlockwiseOp().initialize(f, c["B"], c["H"], c["W"], c["stride"], xs[i], os_[i]) for i in range(NBc)]
    stream = torch.cuda.current_stream()
    for i in range(warmup):
        ops[i % NBc](stream)
    torch.cuda.synchronize()
    from shflbw_sparse_nn_b200 import _cabi
    import ctypes as C
    lib = _cabi.lib()
    run_steps, G = capture_steps(torch, lambda i, raw: lib.shflbw_spconv_exec(C.byref(ops[i % NBc]._state), raw), steps,
                                 stream, use_graph=use_graph)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    run_steps()
    e1.record(stream)
    torch.cuda.synchronize()
    f.device_status()
    t = e0.elapsed_time(e1) * 1e-3 / steps
    npix = c["B"] * c["H"] * c["W"]
    flops = 2.0 * f.nnzb * V_ * npix
    byt = 2 * f.nnzb * V_ + 4 * f.nnzb + 4 * (c["F"] // V_ + 1) + 4 * c["F"] + 2 * npix * c["C"] + 2 * npix * c["F"]
    t_roof = max(flops / (pk["tflops"] * 1e12), byt / (pk["hbm_gbs"] * 1e9))
    return {"workload": "SpConv NHWC 16x14x14x512 -> 2048, 3x3 s1 p1, V=64 density=0.1 filter-permute",
            "us_per_call": round(t * 1e6, 3), "img_per_s": round(c["B"] / t, 1), "nonzero_tflops": round(flops / t / 1e12, 3),
            "dense_equivalent_tflops": round(2.0 * npix * c["C"] * c["R"] * c["S"] * c["F"] / t / 1e12, 2),
            "launches_per_call": ops[0].launches_per_exec, "launch": (f"CUDA graph of {G} calls" if G else "host launches"), "t_roof_us": round(t_roof * 1e6, 3),
            "roofline_frac": round(t_roof / t, 4), "algorithmic_bytes": byt, "nnzb": f.nnzb}


def bench_reference_gpu(sb, torch, m, Bd, Dd):
    """The reference's CUDA kernels (built for sm_100a from its own sources) on the same arrays,
    with its own protocol: 10 warm-up + 100 timed launches between two events."""
    sys.path.insert(0, str(ROOT / "tests"))
    try:
        import oracle_api as oa
    except Exception as e:  # pragma: no cover
        return {"unavailable": str(e)}
    if oa.ref_gpu() is None:
        return {"unavailable": "oracle/_ref/libshflbw_ref_gpu.so not built"}
    perm = m.row_permute_ids
    res = {}
    for cfg, name in oa.ref_gpu_spmm_configs(V_):
        rc, ms = oa.ref_gpu_spmm(cfg, M_, K_, N_, V_, m.indptr, m.indices, m.values, perm, Bd.data_ptr(), Dd.data_ptr(), 10, 100)
        res[name] = round(ms * 1e3, 2) if rc == 0 else f"rc={rc}"
    ok = {k: v for k, v in res.items() if isinstance(v, float)}
    best = min(ok, key=ok.get) if ok else None
    return {"us_per_launch": res, "best": best, "best_us": ok.get(best) if best else None,
            "note": "single B/D pair (L2-warm), reference timing protocol"}


_CPU_B_CACHE = {}


def cpu_baseline_sample(m, threads: int, budget_s: float, t_probe: float = 0.0):
    """Times the reference's CPU check (oracle/_ref, unmodified get_host_reference; the oracle
    port if that build is absent) on a column slice of the workload sized for ~budget_s."""
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_api as oa
    import shflbw_sparse_nn_b200 as sb
    use_ref = oa.ref_host() is not None
    perm = m.row_permute_ids
    indptr, indices, values = m.indptr, m.indices, m.values

    def run(ncols, seed):
        B = _CPU_B_CACHE.get((seed, ncols))
        if B is None:                        # inputs are built outside the timed part and reused
            B = _CPU_B_CACHE[(seed, ncols)] = sb.uniform_half(seed, K_ * ncols).reshape(K_, ncols)
        t0 = time.perf_counter()
        if use_ref:
            oa.ref_spmm_host_reference(M_, K_, ncols, V_, indptr, indices, values, perm, B)
        else:
            oa.spmm_ref(M_, ncols, V_, indptr, indices, values, perm, B, threads=1)
        return time.perf_counter() - t0

    if t_probe <= 0.0:
        t_probe = run(32, 1)                 # ~0.2 s for 32 columns: sizes the sample
    per_thread = max(8, int(budget_s / max(t_probe, 1e-3) * 32) // 8 * 8)
    per_thread = min(per_thread, N_)
    times = [0.0] * threads
    def work(i):
        times[i] = run(per_thread, 10 + i)
    ths = [threading.Thread(target=work, args=(i,)) for i in range(threads)]
    t0 = time.perf_counter()
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    wall = time.perf_counter() - t0
    cols = per_thread * threads
    nnz = m.nnzb * V_
    return {"value": round(2.0 * nnz * cols / wall / 1e12, 6), "unit": UNIT, "cores": threads,
            "kind": "reference" if use_ref else "port",
            "sample": f"{cols} dense columns of the {N_}-column workload ({per_thread} per thread), {wall:.2f} s wall",
            "seconds": round(wall, 3), "t_probe": t_probe}


def run_reference(args):
    """Reference arm: the reference's CPU implementation of the path on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import shflbw_sparse_nn_b200 as sb
    m = build_problem(sb)
    threads = os.cpu_count() or 1
    W = max(1, min(args.warmup, 1))
    steps = max(1, args.steps)
    # whole run within a few minutes whatever K is (the sample is sized from a single-thread
    # probe; all threads together run it ~2x slower)
    budget = min(8.0, 90.0 / (steps + W))
    probe = 0.0
    for _ in range(W):
        probe = cpu_baseline_sample(m, threads, budget_s=min(budget, 1.0), t_probe=probe)["t_probe"]
    vals, secs, sample = [], [], None
    for _ in range(steps):
        r = cpu_baseline_sample(m, threads, budget_s=budget, t_probe=probe)
        vals.append(r["value"]); secs.append(r["seconds"]); sample = r
    value = statistics.mean(vals)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    out = {"impl": "reference", "metric": METRIC, "value": round(value, 6), "unit": UNIT, "n_gpus": world,
           "steps": steps, "warmup": W, "ms_per_step": round(statistics.mean(secs) * 1e3, 3),
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": "SpMM M=N=K=4096 V=64 density=0.1 row-permute seed=2021 fp16 uniform[-1,1)",
                      "note": "reference CPU check (get_host_reference), each step a column slice of the workload"},
           "cpu_baseline": {"value": round(value, 6), "unit": UNIT, "cores": threads, "kind": sample["kind"],
                            "sample": sample["sample"]},
           "e2e": {"value": round(value, 6), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch every timed step from the host instead of replaying a CUDA graph")
    ap.add_argument("--quick", action="store_true",
                    help="profiling aid: timed SpMM loop plus a short SpConv loop only (no e2e, no reference kernels, no CPU baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
