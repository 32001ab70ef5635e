"""Shape sweeps on one GPU: the counterpart of the reference's sweep scripts
(scripts/benchmark/gemm.block_sparse.sh, scripts/benchmark/conv.block_sparse.sh), which loop
benchmark.spmm.out / benchmark.spconv.out over lists of shapes.

    python -m shflbw_sparse_nn_b200.sweep spmm      [--reps 50] [--json out.json]
    python -m shflbw_sparse_nn_b200.sweep resnet50  [--batch 256] [--reps 20] [--chained] [--json out.json]

`spmm` walks transformer projection shapes x N x V x density with seeded masks and uniform
values and prints, per shape, the time, nonzero and dense-equivalent TFLOP/s and the fraction
of the per-shape roofline (slower of nonzero FLOPs at the tensor peak and compulsory bytes at
the HBM peak).  `resnet50` times every pruned 1x1 / 3x3 layer shape of the ResNet-50 topology
(V=64, density 0.2) at the given batch and reports images/s over the pruned layers of one
forward pass (each distinct shape weighted by how often the [3,4,6,3] stack uses it; the dense
7x7 stem and the pooling / classifier layers are not part of the sparse path and not timed).
With --chained every layer runs as a chained layer (activations stay channel-major, halo-padded
and in stored filter order between layers; one launch per layer, ReLU fused).  Launched with
`python -m torch.distributed.run --nproc-per-node G --master-addr 127.0.0.1 -m
shflbw_sparse_nn_b200.sweep resnet50 ...` the batch is split over G GPUs (filters replicated, no
exchange) and the per-layer time is the maximum over the ranks.

Timing follows the reference's tool (benchmark/benchmark.spmm.cu:36-49): warm-up launches,
then the mean over `reps` launches between two CUDA events (the launches replayed from one CUDA
graph, so that small kernels are not hidden behind the host's launch cost).  Inputs alternate between buffers
whose total size exceeds the L2 cache.  Peaks come from --hbm-gbs / --tflops (defaults: a measured
copy bandwidth and dense fp16 tensor throughput of one B200)."""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

SPMM_WEIGHTS = [(3072, 768), (768, 3072), (4096, 4096), (11008, 4096)]
SPMM_N = [512, 4096, 16384]
SPMM_V = [16, 32, 64, 128]
SPMM_DENSITY = [0.05, 0.1, 0.25, 0.5]

# (Hout, Wout, C, F, R, S, stride, uses in one forward pass of the [3,4,6,3] bottleneck stack)
RESNET50_LAYERS = [
    (56, 56, 64, 64, 1, 1, 1, 1), (56, 56, 256, 64, 1, 1, 1, 2), (56, 56, 64, 64, 3, 3, 1, 3),
    (56, 56, 64, 256, 1, 1, 1, 4), (56, 56, 256, 128, 1, 1, 1, 1), (28, 28, 512, 128, 1, 1, 1, 3),
    (28, 28, 128, 128, 3, 3, 2, 1), (28, 28, 128, 128, 3, 3, 1, 3), (28, 28, 128, 512, 1, 1, 1, 4),
    (28, 28, 256, 512, 1, 1, 2, 1), (28, 28, 512, 256, 1, 1, 1, 1), (14, 14, 1024, 256, 1, 1, 1, 5),
    (14, 14, 256, 256, 3, 3, 2, 1), (14, 14, 256, 256, 3, 3, 1, 5), (14, 14, 256, 1024, 1, 1, 1, 6),
    (14, 14, 512, 1024, 1, 1, 2, 1), (14, 14, 1024, 512, 1, 1, 1, 1), (7, 7, 2048, 512, 1, 1, 1, 2),
    (7, 7, 512, 512, 3, 3, 2, 1), (7, 7, 512, 512, 3, 3, 1, 2), (7, 7, 512, 2048, 1, 1, 1, 3),
    (7, 7, 1024, 2048, 1, 1, 2, 1),
]

L2_BYTES = 126 << 20


def _time(torch, launches, reps, warmup=5):
    """Mean seconds per launch: `reps` launches (rotating through `launches`) captured once into a
    CUDA graph and replayed, so that the host's per-launch cost does not hide kernels of a few
    microseconds; falls back to plain launches if capture is not possible."""
    s = torch.cuda.current_stream()
    for i in range(warmup):
        launches[i % len(launches)](s)
    torch.cuda.synchronize()
    run = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                cap = torch.cuda.current_stream()
                for i in range(reps):
                    launches[i % len(launches)](cap)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        run = graph.replay
    except Exception:
        torch.cuda.synchronize()
        run = lambda: [launches[i % len(launches)](s) for i in range(reps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s)
    run()
    e1.record(s)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps  # seconds


def _roof(flops, nbytes, args):
    return max(flops / (args.tflops * 1e12), nbytes / (args.hbm_gbs * 1e9))


def sweep_spmm(args, sb, torch):
    rows = []
    gen = torch.Generator(device="cuda").manual_seed(7)
    for (M, K) in SPMM_WEIGHTS:
        for V in SPMM_V:
            for d in SPMM_DENSITY:
                m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, d, True, 2021, values="uniform")
                m.transform_and_sync_device()
                for N in SPMM_N:
                    if args.max_n and N > args.max_n:
                        continue
                    per = 2 * (K + M) * N
                    nb = max(2, min(8, -(-L2_BYTES // per) + 1))
                    Bs = [(torch.rand((K, N), generator=gen, device="cuda") * 2 - 1).half() for _ in range(nb)]
                    Ds = [torch.empty((M, N), dtype=torch.float16, device="cuda") for _ in range(nb)]
                    ops = [sb.SpmmBlockwiseOp().initialize(m, N, Bs[i], Ds[i]) for i in range(nb)]
                    t = _time(torch, ops, args.reps)
                    m.device_status()
                    flops = 2.0 * m.nnzb * V * N
                    nbytes = 2 * m.nnzb * V + 4 * m.nnzb + 4 * (M // V + 1) + 4 * M + 2 * K * N + 2 * M * N
                    row = dict(M=M, K=K, N=N, V=V, density=d, nnzb=m.nnzb, us=t * 1e6, nonzero_tflops=flops / t / 1e12,
                               dense_equiv_tflops=2.0 * M * K * N / t / 1e12, roofline_frac=_roof(flops, nbytes, args) / t,
                               tile=ops[0]._state.tokens_per_cta)
                    rows.append(row)
                    print("spmm M={M:5d} K={K:5d} N={N:5d} V={V:3d} d={density:.2f}: {us:8.1f} us  {nonzero_tflops:7.1f} nz-TFLOP/s  "
                          "{dense_equiv_tflops:8.1f} dense-eq  roofline {roofline_frac:.3f}  tile {tile}".format(**row), flush=True)
                    del ops, Bs, Ds
                del m
    return rows


def sweep_resnet50(args, sb, torch):
    """Under torchrun (WORLD_SIZE > 1, one rank per GPU) the batch is split evenly over the ranks
    -- the path shards along the batch with the filters replicated and no exchange -- and every
    layer's time is the maximum over the ranks; rank 0 prints."""
    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
        if args.batch % world:
            raise SystemExit("--batch must be divisible by the number of ranks")
    rows, total = [], 0.0
    gen = torch.Generator(device="cuda").manual_seed(11 + rank)
    Bn = args.batch // world
    for (Ho, Wo, Cc, F, R, S, stride, uses) in RESNET50_LAYERS:
        Hin, Win = Ho * stride, Wo * stride
        f = sb.BlockwiseSpFilter().init_random(F, R, S, Cc, 64, 1, 0.2, True, 2021, values="uniform")
        f.transform_and_sync_device()
        per = 2 * Bn * (Hin * Win * Cc + Ho * Wo * F)
        nb = max(2, min(4, -(-L2_BYTES // per) + 1))
        xs = [(torch.rand((Bn, Hin, Win, Cc), generator=gen, device="cuda") * 2 - 1).half() for _ in range(nb)]
        os_ = [torch.empty((Bn, Ho, Wo, F), dtype=torch.float16, device="cuda") for _ in range(nb)]
        if args.chained:
            # activations stay in the chain-buffer layout: one launch per layer, ReLU fused,
            # output halo sized for a 3x3 consumer (the larger of the two cases in this stack)
            del xs, os_
            ins = [torch.zeros(sb.chain_buffer_elems(Cc, Hin, Win, Bn, R, S), dtype=torch.float16, device="cuda")
                   for _ in range(nb)]
            for b_ in ins:
                b_.view(Cc, -1)[:, :].uniform_(-1, 1, generator=gen)   # halo values do not affect the timing
            xs = ins
            os_ = [torch.zeros(sb.chain_buffer_elems(F, Ho, Wo, Bn, 3, 3), dtype=torch.float16, device="cuda")
                   for _ in range(nb)]
            ops = [sb.SpconvChainOp().initialize(f, Bn, Hin, Win, stride, xs[i], os_[i], 3, 3, relu=True)
                   for i in range(nb)]
        else:
            ops = [sb.SpconvBlockwiseOp().initialize(f, Bn, Hin, Win, stride, xs[i], os_[i]) for i in range(nb)]
        if dist:
            dist.barrier()
        t = _time(torch, ops, args.reps)
        f.device_status()
        if dist:
            tt = torch.tensor([t], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        flops = 2.0 * f.nnzb * 64 * Bn * Ho * Wo
        nbytes = 2 * f.nnzb * 64 + 4 * f.nnzb + 4 * (F // 64 + 1) + 4 * F + per
        row = dict(Ho=Ho, Wo=Wo, C=Cc, F=F, R=R, S=S, stride=stride, uses=uses, batch=Bn, us=t * 1e6,
                   nonzero_tflops=flops / t / 1e12, roofline_frac=_roof(flops, nbytes, args) / t,
                   tile=ops[0]._state.tokens_per_cta)
        rows.append(row)
        total += t * uses
        if rank == 0:
            print("conv {Ho:3d}x{Wo:<3d} C={C:5d} F={F:5d} {R}x{S}/{stride} x{uses}: {us:9.1f} us  {nonzero_tflops:7.1f} nz-TFLOP/s  "
                  "roofline {roofline_frac:.3f}  tile {tile}".format(**row), flush=True)
        del ops, xs, os_, f
    summary = dict(batch=args.batch, gpus=world, batch_per_gpu=Bn, chained=bool(args.chained), pruned_layers_ms=total * 1e3,
                   images_per_s=args.batch / total)
    if rank == 0:
        print("resnet50 pruned layers, batch {batch} over {gpus} GPU(s), chained={chained}: {pruned_layers_ms:.3f} ms per forward pass "
              "-> {images_per_s:.0f} images/s".format(**summary), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    return rows + [summary]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("which", choices=["spmm", "resnet50"])
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--max-n", type=int, default=0, help="spmm: skip dense widths above this")
    ap.add_argument("--chained", action="store_true",
                    help="resnet50: time every layer as a chained layer (chain buffers in and out, one launch)")
    ap.add_argument("--hbm-gbs", type=float, default=6460.5)
    ap.add_argument("--tflops", type=float, default=1632.1)
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)
    import torch

    import shflbw_sparse_nn_b200 as sb
    if not torch.cuda.is_available():
        print("sweep: no CUDA device", file=sys.stderr)
        return 2
    rows = sweep_spmm(args, sb, torch) if args.which == "spmm" else sweep_resnet50(args, sb, torch)
    if args.json and int(__import__("os").environ.get("RANK", "0")) == 0:
        with open(args.json, "w") as fh:
            json.dump(dict(which=args.which, hbm_gbs=args.hbm_gbs, tflops=args.tflops, rows=rows), fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
