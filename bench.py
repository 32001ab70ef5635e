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

The K timed steps are repeated as R blocks (R chosen so that the timed region lasts at least
50 ms); every block is bracketed by CUDA events on the launching stream, the whole region by a
barrier and a device synchronisation; `ms_per_step` is the median over blocks of the
max-over-ranks block time divided by K, and the spread is printed beside it.

Printed JSON (one line, rank 0):
  value      nonzero-only TFLOP/s (2 * nnz * N / t), inputs resident in HBM
  dense_equivalent_tflops   2*M*K*N / t (what the reference's tool prints as "effective")
  roofline   achieved algorithmic GB/s of the SpMM kernel against the measured HBM peak
  e2e        same metric through the host-buffer C-ABI call (H2D + kernel + D2H per step), with the
             time of the bare copies (same buffers, streams and chunks, no kernel) beside it
  spconv     the headline SpConv (16x14x14x512 -> 2048, 3x3) on every GPU, images/s summed
  resnet50   the ResNet-50-shaped stack of 52 chained sparse convolutions executed as one forward
             pass (CUDA graph), batch 256 split over the GPUs (strong scaling), images/s
  with_gather  (N > 1) the SpMM step followed by an all-gather of the output shards
  cpu_baseline  the reference's CPU check timed on this box on a column slice
  reference_gpu_kernel  the reference's own CUDA kernels (sm_100a build) on the same inputs, L2-cold

--impl reference times the reference's CPU implementation (oracle/_ref) on all host threads.
"""
from __future__ import annotations

import argparse
import json
import math
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
RESNET_BATCH = 256
METRIC = "spmm_nonzero_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "SpMM M=N=K=4096 V=64 density=0.1 row-permute seed=2021 fp16 uniform[-1,1)"
MIN_TIMED_MS = 50.0


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), tflops=float(d["bf16_tflops"]),
                    tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def ncu_traffic():
    """DRAM bytes (read + write) of one SpMM launch on this workload, from the ncu capture whose
    summary sits beside this number; None when no capture of the current kernel is recorded."""
    p = ROOT / "profiles" / "panel_umma_spmm_4096_v64.json"
    try:
        d = json.loads(p.read_text())
        return int(d["dram_bytes_read_per_launch"]) + int(d["dram_bytes_written_per_launch"]), d.get("kernel")
    except Exception:
        return None, None


def ncu_spconv_shares():
    """Share of each of the three launches of an NHWC SpConv call (planes-out plan) in the call's
    device time, from the ncu launch list summarised under profiles/ (cold-cache, serialised);
    None when no record is there."""
    p = ROOT / "profiles" / "panel_umma_spconv_16x14x14x512.json"
    try:
        return json.loads(p.read_text())["share_of_the_call"]
    except Exception:
        return None


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


class Dist:
    """torch.distributed plumbing: barrier and max-over-ranks only (no collective on the data path)."""

    def __init__(self, torch):
        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.pg = None
        torch.cuda.set_device(self.local)
        if self.world > 1:
            import torch.distributed as dist
            # The collectives here are a barrier, a max over a few doubles and one optional all-gather:
            # nothing that needs in-switch reduction, so NCCL's NVLink-multicast set-up is left out
            # unless the caller asks for it (one 4-GPU run on a shared box never got past NCCL's
            # initialisation).  A rendezvous or collective that does not complete ends the run with
            # an error after three minutes instead of the default ten.
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            import datetime
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local),
                                    timeout=datetime.timedelta(seconds=180))
            self.pg = dist

    def barrier(self):
        if self.pg:
            self.pg.barrier()
        self.torch.cuda.synchronize()

    def max(self, values):
        """Element-wise maximum over ranks of a list of floats."""
        if not self.pg:
            return list(values)
        t = self.torch.tensor(list(values), device="cuda", dtype=self.torch.float64)
        self.pg.all_reduce(t, op=self.pg.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.pg:
            self.pg.barrier()
            self.pg.destroy_process_group()


def capture_steps(torch, launch, steps, stream, use_graph=True):
    """Capture G consecutive steps (G = largest divisor of `steps` up to 200) into a CUDA graph.
    Returns (run, G, est): run() executes exactly `steps` steps on `stream`; G == 0 means plain
    launches; est = measured ms per step of a short untimed run (one graph replay, or up to 200 plain
    launches -- not the whole block, so that the timed region is not preceded by a run as long as
    itself).  launch(i, raw_stream) enqueues step i."""
    G = max((g for g in range(1, min(steps, 200) + 1) if steps % g == 0), default=0) if use_graph else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if G < 2:
        n = min(steps, 200)
        e0.record(stream)
        for i in range(n):
            launch(i, stream.cuda_stream)
        e1.record(stream)
        torch.cuda.synchronize()
        return (lambda: [launch(i, stream.cuda_stream) for i in range(steps)]), 0, e0.elapsed_time(e1) / n
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
    e0.record(stream)
    graph.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    return (lambda: [graph.replay() for _ in range(steps // G)]), G, e0.elapsed_time(e1) / G


def timed_blocks(torch, dist, run_block, steps, est_ms_per_step, stream):
    """R blocks of `steps` steps, each between two events on `stream`; the region between a barrier
    and a synchronisation on both sides.  Returns (median ms per step, min, max, R, wall t0, t1):
    per block the time is the maximum over ranks."""
    R = max(1, min(400, math.ceil(MIN_TIMED_MS / max(est_ms_per_step * steps, 1e-4))))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(R + 1)]
    dist.barrier()
    t0 = time.time()
    ev[0].record(stream)
    for r in range(R):
        run_block()
        ev[r + 1].record(stream)
    torch.cuda.synchronize()
    t1 = time.time()
    dist.barrier()
    per_block = dist.max([ev[r].elapsed_time(ev[r + 1]) for r in range(R)])
    per_step = sorted(b / steps for b in per_block)
    return statistics.median(per_step), per_step[0], per_step[-1], R, t0, t1


def build_problem(sb):
    return sb.BlockwiseSpMatrix().init_random(M_, K_, V_, 1, DENSITY, True, SEED, values="uniform")


def run_ours(args):
    import ctypes as C

    import torch

    import shflbw_sparse_nn_b200 as sb
    from shflbw_sparse_nn_b200 import _cabi
    from shflbw_sparse_nn_b200.build import build_library

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    dist = Dist(torch)
    world, rank, local = dist.world, dist.rank, dist.local
    if rank == 0:
        build_library()
    dist.barrier()
    lib = _cabi.lib()

    pk = peaks()
    if args.only == "spconv":       # profiling aid: the SpConv loop alone
        out = {"spconv": bench_spconv(sb, torch, dist, pk, steps=args.steps, warmup=max(3, args.warmup), use_graph=not args.no_graph)}
        dist.close()
        if rank == 0:
            print(json.dumps(out))
        return
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
    states = [C.byref(op._state) for op in ops]
    stream = torch.cuda.current_stream()

    def launch(i, raw):
        lib.shflbw_spmm_exec(states[i % NB], raw)

    W = max(3, args.warmup)
    sampler = ClockSampler(local) if rank == 0 else None
    time.sleep(0.05)
    for i in range(W):
        launch(i, stream.cuda_stream)
    torch.cuda.synchronize()

    # The timed loop is launch-gap sensitive (a kernel of a few tens of microseconds per step):
    # consecutive steps are captured once into a CUDA graph and the graph is replayed.
    run_steps, G, est = capture_steps(torch, launch, args.steps, stream, use_graph=not args.no_graph)
    ms_step, ms_lo, ms_hi, R, t_wall0, t_wall1 = timed_blocks(torch, dist, run_steps, args.steps, est, stream)
    m.device_status()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    value = world * flops_nz / (ms_step * 1e-3) / 1e12

    t_kernel = ms_step * 1e-3  # one kernel per step, launched back to back on one stream
    t_tc, t_hbm = flops_nz / (pk["tflops"] * 1e12), bytes_alg / (pk["hbm_gbs"] * 1e9)
    bound = "hbm" if t_hbm >= t_tc else "tensor"
    if bound == "hbm":
        achieved, peak, runit = bytes_alg / t_kernel / 1e9, pk["hbm_gbs"], "GB/s"
    else:
        achieved, peak, runit = flops_nz / t_kernel / 1e12, pk["tflops"], "TFLOP/s"
    st0 = ops[0]._state
    kernel_name = (f"panel_umma_kernel<V={V_},T={st0.tokens_per_cta},stages={st0.stages},producers={st0.producer_warps},"
                   f"{'rows' if st0.variant else 'tokens'}-in-lanes,{'tma-gather4' if st0.gather else 'cp.async'}>")
    traffic, traffic_kernel = ncu_traffic()
    roofline = {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": runit,
                "frac": round(achieved / peak, 4), "traffic": traffic, "traffic_captured_on": traffic_kernel,
                "peak_source": pk["source"], "algorithmic_bytes": bytes_alg, "algorithmic_flops": flops_nz,
                "kernel": kernel_name, "kernel_us": round(t_kernel * 1e6, 3),
                "t_roof_us": round(max(t_tc, t_hbm) * 1e6, 3), "frac_of_tensor_peak": round(flops_nz / t_kernel / 1e12 / pk["tflops"], 4)}

    out = {
        "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": W,
        "ms_per_step": round(ms_step, 6), "ms_per_step_min": round(ms_lo, 6), "ms_per_step_max": round(ms_hi, 6),
        "repeats": R, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "nnzb": nnzb, "batches_rotated": NB, "l2": "inputs larger than L2 (4 x 67 MB rotated)",
                   "per_gpu": "one 4096-column batch per step on every GPU; sparse operand replicated",
                   "timing": f"{R} blocks of {args.steps} steps, median block (max over ranks) / steps",
                   "launch": (f"CUDA graph of {G} steps replayed {args.steps // G}x per block" if G else "one host launch per step"),
                   "power": ("a timed region of ~60 ms runs at the full SM clock; 100+ ms of back-to-back launches of this "
                             "kernel reach the board's power cap (sw_power_cap, ~1.85-1.89 GHz measured: ~36.7 us per step)")},
        "dense_equivalent_tflops": round(world * flops_dense / (ms_step * 1e-3) / 1e12, 2),
        "roofline": roofline, "gpu_launches": R * args.steps * ops[0].launches_per_exec, "clocks": clocks,
    }

    # ---- SpConv and the executed ResNet-50 stack, at every N ----
    out["spconv"] = bench_spconv(sb, torch, dist, pk, steps=60 if args.quick else 300, warmup=10,
                                 use_graph=not args.no_graph)
    if not args.quick:
        try:
            out["resnet50"] = bench_resnet50(torch, dist)
        except Exception as e:  # pragma: no cover - reported, never hidden
            out["resnet50"] = {"error": f"{type(e).__name__}: {e}"[:300]}

    if args.quick:
        dist.close()
        if rank == 0:
            print(json.dumps(out))
        return

    # ---- N > 1: the same step followed by an all-gather of the output shards ----
    if world > 1:
        out["with_gather"] = bench_with_gather(torch, dist, launch, Ds, flops_nz)

    # ---- end to end through the host-buffer C-ABI call (H2D + kernel + D2H inside the timing) ----
    e2e_steps = max(3, min(args.steps, 10))
    Bh = torch.from_numpy(sb.uniform_half(500 + rank, K_ * N_).reshape(K_, N_).view(np.int16)).pin_memory()
    Dh = torch.zeros((M_, N_), dtype=torch.int16).pin_memory()

    def host_loop(fn):
        for _ in range(2):
            fn()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            fn()                              # synchronous: returns after the D2H copy completed
        t = (time.perf_counter() - t0) / e2e_steps
        dist.barrier()
        return dist.max([t])[0]

    t_e2e = host_loop(lambda: sb.spmm_host(m, N_, Bh, Dh))
    t_floor = host_loop(lambda: _cabi.check(lib.shflbw_spmm_host_copies_only(m._h, N_, Bh.data_ptr(), Dh.data_ptr(), 0), "copies"))
    t_floor_c = host_loop(lambda: _cabi.check(lib.shflbw_spmm_host_copies_only(m._h, N_, Bh.data_ptr(), Dh.data_ptr(), 1), "copies"))
    out["e2e"] = {"value": round(world * flops_nz / t_e2e / 1e12, 4), "unit": UNIT,
                  "h2d_bytes_per_step": 2 * K_ * N_, "d2h_bytes_per_step": 2 * M_ * N_,
                  "ms_per_step": round(t_e2e * 1e3, 4), "steps": e2e_steps,
                  "copy_floor_ms": round(t_floor * 1e3, 4), "copy_floor_contiguous_ms": round(t_floor_c * 1e3, 4),
                  "over_copy_floor": round(t_e2e / t_floor, 3),
                  "aggregate_link_gbs": round(world * (2 * K_ * N_ + 2 * M_ * N_) / t_floor / 1e9, 1),
                  "call": "shflbw_spmm_host (pinned host B and D); copy floor = the same copies, streams and chunks without the kernel",
                  "host": host_topology(local)}

    if rank == 0 and world == 1:
        out["reference_gpu_kernel"] = bench_reference_gpu(sb, torch, m, Bs, Ds)
        ref_best = out["reference_gpu_kernel"].get("spmm", {}).get("best_us")
        if ref_best:
            out["speedup_over_reference_gpu_kernel"] = {"spmm": round(ref_best / (ms_step * 1e3), 3)}
            cbest = out["reference_gpu_kernel"].get("spconv", {}).get("best_us")
            if cbest and "us_per_call" in out["spconv"]:
                out["speedup_over_reference_gpu_kernel"]["spconv"] = round(cbest / out["spconv"]["us_per_call"], 3)
        out["cpu_baseline"] = cpu_baseline_sample(m.indptr, m.indices, m.values, m.row_permute_ids, m.nnzb, threads=1, budget_s=12.0)
        out["cpu_baseline"].pop("t_probe", None)
    dist.close()
    if rank == 0:
        print(json.dumps(out))


def host_topology(local):
    """What the host side of the copies looks like from this rank: CPU set and NUMA node of the GPU."""
    info = {"cpus_allowed": len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else None}
    try:
        q = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(local)],
                           capture_output=True, text=True, timeout=10).stdout.strip()
        bus = q.lower()
        if bus.startswith("00000000:"):
            bus = "0000:" + bus[9:]
        node = Path(f"/sys/bus/pci/devices/{bus}/numa_node")
        info["gpu_numa_node"] = int(node.read_text()) if node.exists() else None
    except Exception:
        info["gpu_numa_node"] = None
    return info


def bench_spconv(sb, torch, dist, pk, steps=300, warmup=20, use_graph=True):
    """Config 3 on every rank (weak scaling: 16 images per call per GPU), images/s summed over ranks."""
    import ctypes as C
    from shflbw_sparse_nn_b200 import _cabi
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
    lib = _cabi.lib()
    run_steps, G, est = capture_steps(torch, lambda i, raw: lib.shflbw_spconv_exec(C.byref(ops[i % NBc]._state), raw), steps,
                                 stream, use_graph=use_graph)
    ms, lo, hi, R, _, _ = timed_blocks(torch, dist, run_steps, steps, est, stream)
    f.device_status()
    t = ms * 1e-3
    npix = c["B"] * c["H"] * c["W"]
    flops = 2.0 * f.nnzb * V_ * npix
    byt = 2 * f.nnzb * V_ + 4 * f.nnzb + 4 * (c["F"] // V_ + 1) + 4 * c["F"] + 2 * npix * c["C"] + 2 * npix * c["F"]
    t_roof = max(flops / (pk["tflops"] * 1e12), byt / (pk["hbm_gbs"] * 1e9))
    st = ops[0]._state
    return {"workload": "SpConv NHWC 16x14x14x512 -> 2048, 3x3 s1 p1, V=64 density=0.1 filter-permute; every GPU runs it on its own images",
            "us_per_call": round(t * 1e6, 3), "us_min": round(lo * 1e3, 3), "us_max": round(hi * 1e3, 3),
            "img_per_s": round(dist.world * c["B"] / t, 1), "n_gpus": dist.world,
            "nonzero_tflops": round(dist.world * flops / t / 1e12, 3),
            "dense_equivalent_tflops": round(dist.world * 2.0 * npix * c["C"] * c["R"] * c["S"] * c["F"] / t / 1e12, 2),
            "launches_per_call": ops[0].launches_per_exec,
            "plan": "planes out (filters in TMEM lanes) + transpose" if st.variant == 1 else "positions out (tokens in TMEM lanes)",
            "launch": (f"CUDA graph of {G} calls" if G else "host launches"), "repeats": R,
            "t_roof_us": round(t_roof * 1e6, 3), "roofline_frac": round(t_roof / t, 4), "algorithmic_bytes": byt, "nnzb": f.nnzb,
            "launch_shares_ncu": ncu_spconv_shares() if st.variant == 1 else None}


def bench_resnet50(torch, dist):
    """The 52 pruned convolutions of ResNet-50 executed as one forward pass (import, chained layers
    with folded channel orders, residual adds and ReLU fused, export), batch 256 split over the
    ranks; one CUDA graph per rank; images/s of the whole job."""
    from shflbw_sparse_nn_b200.resnet50 import SparseResNet50
    if RESNET_BATCH % dist.world:
        return {"skipped": f"batch {RESNET_BATCH} does not split over {dist.world} ranks"}
    Bn = RESNET_BATCH // dist.world
    net = SparseResNet50(Bn, hw=56, density=0.2, V=64, seed=SEED)
    net.x.uniform_(-1, 1)
    replay = net.capture()
    stream = torch.cuda.current_stream()
    for _ in range(3):
        replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    replay()
    e1.record(stream)
    torch.cuda.synchronize()
    est = e0.elapsed_time(e1)
    ms, lo, hi, R, _, _ = timed_blocks(torch, dist, replay, 1, est, stream)
    net.check_status()
    finite = bool(torch.isfinite(net.y.float()).all().item())
    flops = net.nonzero_flops() * dist.world
    return {"workload": "ResNet-50 pruned convolutions (52 layers, V=64, density 0.2), 56x56x64 input, executed forward pass",
            "batch": RESNET_BATCH, "batch_per_gpu": Bn, "n_gpus": dist.world, "scaling": "strong",
            "ms_per_forward": round(ms, 4), "ms_min": round(lo, 4), "ms_max": round(hi, 4), "repeats": R,
            "images_per_s": round(RESNET_BATCH / (ms * 1e-3), 1), "nonzero_tflops": round(flops / (ms * 1e-3) / 1e12, 2),
            "launches_per_forward": net.launches_per_forward, "launch": "one CUDA graph per forward pass",
            "output_finite": finite}


def bench_with_gather(torch, dist, launch, Ds, flops_nz):
    """SpMM step + all-gather of the M x 4096 output shards (layout [rank][M][N/ranks-as-owned]),
    for callers that want the full output on every GPU.  Not part of the headline step."""
    stream = torch.cuda.current_stream()
    full = [torch.empty((dist.world,) + tuple(Ds[0].shape), dtype=Ds[0].dtype, device="cuda") for _ in range(2)]
    steps = 20

    def block():
        for i in range(steps):
            launch(i, stream.cuda_stream)
            dist.pg.all_gather_into_tensor(full[i % 2], Ds[i % len(Ds)])
    block()
    torch.cuda.synchronize()
    ms, lo, hi, R, _, _ = timed_blocks(torch, dist, block, steps, 1.0, stream)
    return {"ms_per_step": round(ms, 4), "value": round(dist.world * flops_nz / (ms * 1e-3) / 1e12, 2), "unit": UNIT,
            "gathered_bytes_per_step_per_gpu": int(Ds[0].numel() * 2 * dist.world), "collective": "NCCL all_gather_into_tensor"}


def bench_reference_gpu(sb, torch, m, Bs, Ds):
    """The reference's CUDA kernels (built for sm_100a from its own sources) on the same arrays,
    10 warm-up + 100 timed launches between two events as its tools do, rotating the same buffer
    pairs as the product's timed loop (L2-cold)."""
    sys.path.insert(0, str(ROOT / "tests"))
    try:
        import oracle_api as oa
    except Exception as e:  # pragma: no cover
        return {"unavailable": str(e)}
    if oa.ref_gpu() is None:
        return {"unavailable": "oracle/_ref/libshflbw_ref_gpu.so not built"}
    if not hasattr(oa.ref_gpu(), "ref_gpu_spmm_rotating"):
        return {"unavailable": "oracle/_ref/libshflbw_ref_gpu.so predates the rotating-buffer entry points"}
    perm = m.row_permute_ids
    res = {}
    for cfg, name in oa.ref_gpu_spmm_configs(V_):
        rc, ms = oa.ref_gpu_spmm_rotating(cfg, M_, K_, N_, V_, m.indptr, m.indices, m.values, perm,
                                          [b.data_ptr() for b in Bs], [d.data_ptr() for d in Ds], 10, 100)
        res[name] = round(ms * 1e3, 2) if rc == 0 else f"rc={rc}"
    ok = {k: v for k, v in res.items() if isinstance(v, float)}
    best = min(ok, key=ok.get) if ok else None
    out = {"spmm": {"us_per_launch": res, "best": best, "best_us": ok.get(best) if best else None}}
    # SpConv: the reference's own layouts ([C][H][W][B] in, [F][H][W][B] out); 10 rotating pairs
    c = CONV
    f = sb.BlockwiseSpFilter().init_random(c["F"], c["R"], c["S"], c["C"], V_, 1, DENSITY, True, SEED, values="uniform")
    xs = [torch.rand((c["C"], c["H"], c["W"], c["B"]), device="cuda").half() for _ in range(10)]
    os_ = [torch.zeros((c["F"], c["H"], c["W"], c["B"]), dtype=torch.float16, device="cuda") for _ in range(10)]
    cres = {}
    for cfg, name in oa.ref_gpu_conv_configs(V_):
        rc, ms = oa.ref_gpu_spconv_rotating(cfg, c["B"], c["H"], c["W"], c["C"], c["F"], c["R"], c["S"], c["stride"], V_,
                                            f.indptr, f.indices, f.values, f.row_permute_ids,
                                            [x.data_ptr() for x in xs], [o.data_ptr() for o in os_], 10, 100)
        cres[name] = round(ms * 1e3, 2) if rc == 0 else f"rc={rc}"
    okc = {k: v for k, v in cres.items() if isinstance(v, float)}
    bestc = min(okc, key=okc.get) if okc else None
    out["spconv"] = {"us_per_launch": cres, "best": bestc, "best_us": okc.get(bestc) if bestc else None,
                     "note": "reference layouts [C][H][W][B] -> [F][H][W][B] (no NHWC conversion on its side)"}
    out["note"] = "rotating buffer pairs larger than L2 in aggregate, reference timing protocol (10 + 100 launches)"
    return out


_CPU_B_CACHE = {}


def _uniform_half_np(stream, n):
    """The library's documented seeded fp16 stream (splitmix64 -> uniform[-1, 1)), in numpy, so that
    the reference arm builds its dense operand without loading the product library."""
    with np.errstate(over="ignore"):
        z = (np.uint64(stream) << np.uint64(32)) + np.arange(n, dtype=np.uint64) + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = (z >> np.uint64(40)).astype(np.float64) / float(1 << 24)
    return (2.0 * u - 1.0).astype(np.float32).astype(np.float16)


def cpu_baseline_sample(indptr, indices, values, perm, nnzb, threads: int, budget_s: float, t_probe: float = 0.0):
    """Times the reference's CPU check (oracle/_ref, unmodified get_host_reference; the oracle
    port if that build is absent) on a column slice of the workload sized for ~budget_s."""
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_api as oa
    use_ref = oa.ref_host() is not None

    def run(ncols, seed):
        B = _CPU_B_CACHE.get((seed, ncols))
        if B is None:                        # inputs are built outside the timed part and reused
            B = _CPU_B_CACHE[(seed, ncols)] = _uniform_half_np(seed, K_ * ncols).reshape(K_, ncols)
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
    nnz = nnzb * V_
    return {"value": round(2.0 * nnz * cols / wall / 1e12, 6), "unit": UNIT, "cores": threads,
            "kind": "reference" if use_ref else "port",
            "sample": f"{cols} dense columns of the {N_}-column workload ({per_thread} per thread), {wall:.2f} s wall",
            "seconds": round(wall, 3), "t_probe": t_probe}


def reference_problem():
    """The sparse operand of the workload built WITHOUT the product library: by the reference's own
    builder when oracle/_ref is present, else by the oracle port (both pinned bit-exactly to the
    reference's golden dump); values from the documented seeded stream."""
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_api as oa
    if oa.ref_host() is not None:
        r = oa.RefMatrix.init_random(M_, K_, V_, DENSITY, True, SEED)
        indptr, indices, perm, nnzb = r.indptr, r.indices, r.perm, r.nnzb
    else:
        nnzb, indptr, indices = oa.random_mask(M_, K_, V_, 1, DENSITY, SEED)
        perm = oa.row_permutation(M_, SEED)
    values = _uniform_half_np(SEED, nnzb * V_)
    return indptr, indices, values, perm, nnzb


def run_reference(args):
    """Reference arm: the reference's CPU implementation of the path on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    indptr, indices, values, perm, nnzb = reference_problem()
    threads = os.cpu_count() or 1
    W = max(1, min(args.warmup, 1))
    steps = max(1, args.steps)
    # whole run within a few minutes whatever K is (the sample is sized from a single-thread
    # probe; all threads together run it ~2x slower)
    budget = min(8.0, 90.0 / (steps + W))
    probe = 0.0
    for _ in range(W):
        probe = cpu_baseline_sample(indptr, indices, values, perm, nnzb, threads, budget_s=min(budget, 1.0), t_probe=probe)["t_probe"]
    vals, secs, sample = [], [], None
    for _ in range(steps):
        r = cpu_baseline_sample(indptr, indices, values, perm, nnzb, threads, budget_s=budget, t_probe=probe)
        vals.append(r["value"]); secs.append(r["seconds"]); sample = r
    value = statistics.mean(vals)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    out = {"impl": "reference", "metric": METRIC, "value": round(value, 6), "unit": UNIT, "n_gpus": world,
           "steps": steps, "warmup": W, "ms_per_step": round(statistics.mean(secs) * 1e3, 3),
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": WORKLOAD,
                      "note": "reference CPU check (get_host_reference), each step a column slice of the workload"},
           "cpu_baseline": {"value": round(value, 6), "unit": UNIT, "cores": threads, "kind": sample["kind"],
                            "sample": sample["sample"]},
           "e2e": {"value": round(value, 6), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch every timed step from the host instead of replaying a CUDA graph")
    ap.add_argument("--quick", action="store_true",
                    help="profiling aid: timed SpMM loop plus a short SpConv loop only (no stack, no e2e, no reference kernels, no CPU baseline)")
    ap.add_argument("--only", default="", choices=["", "spconv"],
                    help="profiling aid: run just this part (spconv: the headline SpConv loop with --steps calls)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
