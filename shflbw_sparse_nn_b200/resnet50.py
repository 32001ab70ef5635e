"""ResNet-50-shaped stack of Shfl-BW sparse convolutions, executed as one forward pass.

The 52 pruned convolutions of the [3, 4, 6, 3]-bottleneck topology (every 1x1 and 3x3
convolution after the stem; layer shapes as in the reference's sweep list,
scripts/benchmark/conv.block_sparse.sh:5-27) run as CHAINED layers: activations stay in the
channel-major, halo-padded chain-buffer layout between layers, every layer is one kernel
launch with its scale, residual add and ReLU fused, and the input channels of every filter are
renumbered to the stored filter order of the layer that feeds it.

    x NHWC --import--> [ conv1 1x1 -> conv2 3x3 (/s) -> conv3 1x1 (+ shortcut, ReLU) ] x 16 --export--> y NHWC
                         shortcut = block input, or a 1x1 (/s) projection in the first block of a stage

Weights are random (seeded, uniform[-1, 1) fp16, density 0.2, V = 64 by default): the reference
has no trained checkpoints either, and throughput does not depend on the values.  Each layer's
`alpha` normalises its output (sqrt(6 / non-zeros per row), halved on the residual branch) so
that activations stay inside the fp16 range through all 16 blocks.

The dense 7x7/2 stem and the 3x3/2 max-pool (not pruned in the reference's list either) can be
run in front through torch (`stem=True`): that part is library code, not this package's kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import blockwise as bw

STAGES = ((3, 64, 256, 1), (4, 128, 512, 2), (6, 256, 1024, 2), (3, 512, 2048, 2))   # blocks, mid, out, stride


@dataclass
class LayerSpec:
    name: str
    C: int
    F: int
    R: int
    stride: int
    Hin: int              # input height = width
    src: int              # index of the layer whose output this one reads (-1: the stack's input)
    relu: bool
    residual: Optional[int] = None   # index of the layer whose output is added (-1: the stack's input)
    consumers_R: int = 1  # halo the OUTPUT buffer needs: the largest filter that reads it

    @property
    def Ho(self):
        return -(-self.Hin // self.stride)


def layer_specs(hw: int = 56, c_in: int = 64) -> List[LayerSpec]:
    """The 52 pruned convolutions in execution order, with their data flow."""
    specs: List[LayerSpec] = []
    cur, cur_c, cur_hw = -1, c_in, hw          # producer of the current block input, its channels, its size
    for si, (blocks, mid, out, stride) in enumerate(STAGES):
        for b in range(blocks):
            s = stride if b == 0 else 1
            base = len(specs)
            tag = f"s{si + 1}b{b + 1}"
            shortcut = cur
            if b == 0:   # projection shortcut: 1x1, stride s, no ReLU
                specs.append(LayerSpec(f"{tag}.proj", cur_c, out, 1, s, cur_hw, cur, relu=False))
                shortcut = base
            i1 = len(specs)
            specs.append(LayerSpec(f"{tag}.conv1", cur_c, mid, 1, 1, cur_hw, cur, relu=True, consumers_R=3))
            specs.append(LayerSpec(f"{tag}.conv2", mid, mid, 3, s, cur_hw, i1, relu=True))
            hw2 = -(-cur_hw // s)
            specs.append(LayerSpec(f"{tag}.conv3", mid, out, 1, 1, hw2, i1 + 1, relu=True, residual=shortcut))
            cur, cur_c, cur_hw = i1 + 2, out, hw2
    return specs


class SparseResNet50:
    """Builds the filters, chain buffers and chained ops once; `forward()` enqueues import,
    52 layer launches and export on a stream, `capture()` records that into one CUDA graph."""

    def __init__(self, batch: int, hw: int = 56, density: float = 0.2, V: int = 64, seed: int = 2021,
                 stem: bool = False, device=None):
        import torch

        self.torch = torch
        self.batch, self.hw, self.V, self.density, self.stem = batch, hw, V, density, stem
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.specs = layer_specs(hw)
        dev = self.device
        # stack input and output (NHWC, logical channel order)
        self.x = torch.zeros((batch, hw, hw, 64), dtype=torch.float16, device=dev)
        last = self.specs[-1]
        self.y = torch.zeros((batch, last.Ho, last.Ho, last.F), dtype=torch.float16, device=dev)
        if stem:
            g = torch.Generator(device="cpu").manual_seed(seed)
            self.image = torch.zeros((batch, 3, 4 * hw, 4 * hw), dtype=torch.float16, device=dev).contiguous(
                memory_format=torch.channels_last)
            w = (torch.rand((64, 3, 7, 7), generator=g) * 2 - 1) * math.sqrt(6.0 / 147.0)
            self.stem_w = w.to(dev, torch.float16).contiguous(memory_format=torch.channels_last)
        # filters: logical, then folded to the stored order of the layer that feeds them
        self.filters, self.folded, self.alphas = [], [], []
        for i, sp in enumerate(self.specs):
            f = bw.BlockwiseSpFilter().init_random(sp.F, sp.R, sp.R, sp.C, V, 1, density, True, seed + i, values="uniform")
            self.filters.append(f)
            nnz_row = max(1.0, f.nnzb / (sp.F // V))
            self.alphas.append(math.sqrt(6.0 / nnz_row) * (0.5 if sp.residual is not None else 1.0))
        for i, sp in enumerate(self.specs):
            g_ = self.filters[i] if sp.src < 0 else self.filters[i].fold_input_order(self.filters[sp.src])
            g_.transform_and_sync_device()
            self.folded.append(g_)
        # chain buffers: the stack input (read by 1x1 filters) and one per layer output
        def chain(C_, H, R_):
            return torch.zeros(bw.chain_buffer_elems(C_, H, H, batch, R_, R_), dtype=torch.float16, device=dev)
        self.buf_in = chain(64, hw, 1)
        self.bufs = [chain(sp.F, sp.Ho, sp.consumers_R) for sp in self.specs]
        self.ops = []
        for i, sp in enumerate(self.specs):
            src = self.buf_in if sp.src < 0 else self.bufs[sp.src]
            op = bw.SpconvChainOp().initialize(self.folded[i], batch, sp.Hin, sp.Hin, sp.stride, src, self.bufs[i],
                                               sp.consumers_R, sp.consumers_R, alpha=self.alphas[i], relu=sp.relu)
            if sp.residual is not None:
                res = self.buf_in if sp.residual < 0 else self.bufs[sp.residual]
                op.set_residual(res, None if sp.residual < 0 else self.folded[sp.residual])
            self.ops.append(op)
        self.graph = None

    # ---------------------------------------------------------------------------------
    @property
    def launches_per_forward(self) -> int:
        return 2 + sum(op.launches_per_exec for op in self.ops)

    def nonzero_flops(self) -> float:
        return float(sum(2.0 * f.nnzb * self.V * self.batch * sp.Ho * sp.Ho for f, sp in zip(self.filters, self.specs)))

    def run_stem(self):
        """image [B][3][4hw][4hw] (channels-last) -> self.x [B][hw][hw][64]; torch / cuDNN, not this package's kernels."""
        F = self.torch.nn.functional
        t = F.relu(F.conv2d(self.image, self.stem_w, stride=2, padding=3))
        t = F.max_pool2d(t, 3, stride=2, padding=1)
        self.x.copy_(t.permute(0, 2, 3, 1))

    def forward(self, stream=None):
        """Enqueue one forward pass (self.x -> self.y) on `stream` (a torch stream or None)."""
        if self.stem:
            self.run_stem()
        bw.chain_import_nhwc(self.x, self.batch, self.hw, self.hw, 64, 1, 1, self.buf_in, stream)
        for op in self.ops:
            op(stream)
        last = self.specs[-1]
        bw.chain_export_nhwc(self.bufs[-1], self.batch, last.Ho, last.Ho, last.F, last.consumers_R, last.consumers_R,
                             self.folded[-1], self.y, stream)

    def capture(self):
        """Record forward() into a CUDA graph; returns a callable that replays it."""
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.forward(side)            # warm-up outside the capture (lazy module loads)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                self.forward(torch.cuda.current_stream())
        torch.cuda.synchronize()
        self.graph = graph
        return graph.replay

    def layer_output_nhwc(self, i: int):
        """Output of layer i as an NHWC tensor in logical channel order (for checks)."""
        sp = self.specs[i]
        out = self.torch.zeros((self.batch, sp.Ho, sp.Ho, sp.F), dtype=self.torch.float16, device=self.device)
        bw.chain_export_nhwc(self.bufs[i], self.batch, sp.Ho, sp.Ho, sp.F, sp.consumers_R, sp.consumers_R,
                             self.folded[i], out, None)
        return out

    def check_status(self):
        for f in self.folded:
            f.device_status()
