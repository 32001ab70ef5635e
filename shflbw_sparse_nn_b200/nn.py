"""torch.nn front end: prune a trained `nn.Linear` / `nn.Conv2d` to Shfl-BW and run it through
the library's C ABI on the caller's CUDA stream.

    lin  = ShflBWLinear.from_dense(dense_linear, V=64, density=0.1)     # y = lin(x)
    conv = ShflBWConv2d.from_dense(dense_conv, V=64, density=0.2)       # y = conv(x)

The reference project has no such layer (it only ever builds random patterns,
block_sparse/spmm/blockwise_format.h:70-123, and points to the paper for real models); this
is the piece a user with a trained network needs in front of the hot path.  torch is the
plumbing here (device buffers, the current stream, the bias add and layout views); pruning is
`pruner.prune_matrix` / `prune_conv_filter` on the host, once, and every forward is the
library's SpMM / SpConv kernel.  fp16 inference only; there is no backward pass.
"""
from __future__ import annotations

import numpy as np
import torch
from torch import nn

from . import blockwise as bw
from .pruner import prune_conv_filter, prune_matrix


def _require_cuda_half(x: torch.Tensor, what: str):
    if not x.is_cuda or x.dtype != torch.float16:
        raise TypeError(f"{what}: expected a CUDA float16 tensor, got {x.device} {x.dtype}")


class ShflBWLinear(nn.Module):
    """y = x @ W_pruned^T + b with W in the Shfl-BW format.

    The SpMM computes D[out][tokens] = A[out][in] . B[in][tokens], i.e. it wants activations
    feature-major (tokens contiguous).  `forward` takes the usual [..., in_features] tensor and
    pays one transpose each way; `forward_feature_major` takes [in_features][tokens] and returns
    [out_features][tokens] with no copies (tokens a multiple of 8)."""

    def __init__(self, spmat: bw.BlockwiseSpMatrix, bias: torch.Tensor | None, info: dict | None = None):
        super().__init__()
        self.spmat = spmat
        self.in_features, self.out_features = spmat.ncol, spmat.nrow
        self.info = info or {}
        self.register_buffer("bias", None if bias is None else bias.detach().to(torch.float16))
        self._uploaded_on = None

    @classmethod
    def from_dense(cls, linear: nn.Linear, V: int = 64, density: float = 0.1, permute: bool = True, seed=None):
        m, info = prune_matrix(linear.weight.detach().float().cpu().numpy(), V, density, permute, seed=seed)
        return cls(m, linear.bias, info)

    def _upload(self, device: torch.device):
        if self._uploaded_on != device:
            with torch.cuda.device(device):
                self.spmat.transform_and_sync_device()
            self._uploaded_on = device

    def forward_feature_major(self, xt: torch.Tensor) -> torch.Tensor:
        _require_cuda_half(xt, "ShflBWLinear")
        if xt.dim() != 2 or xt.shape[0] != self.in_features or xt.shape[1] % 8 or not xt.is_contiguous():
            raise ValueError("expected a contiguous [in_features][tokens] tensor with tokens % 8 == 0")
        self._upload(xt.device)
        n = xt.shape[1]
        out = torch.empty((self.out_features, n), dtype=torch.float16, device=xt.device)
        with torch.cuda.device(xt.device):
            op = bw.SpmmBlockwiseOp().initialize(self.spmat, n, xt, out)
            op(torch.cuda.current_stream(xt.device))
        if self.bias is not None:
            out += self.bias.to(xt.device)[:, None]
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _require_cuda_half(x, "ShflBWLinear")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        tokens = x2.shape[0]
        padded = -(-tokens // 8) * 8
        xt = torch.zeros((self.in_features, padded), dtype=torch.float16, device=x.device)
        xt[:, :tokens] = x2.t()
        yt = self.forward_feature_major(xt)
        return yt[:, :tokens].t().reshape(*lead, self.out_features)

    def dense_weight(self) -> torch.Tensor:
        """The pruned weights as a dense [out][in] fp16 tensor (rows in original order), for checks."""
        return torch.from_numpy(densify(self.spmat))


class ShflBWConv2d(nn.Module):
    """Conv2d with a Shfl-BW filter: square odd kernel, padding = kernel // 2, equal strides,
    no dilation or groups, in_channels % 8 == 0, out_channels % V == 0.  Input and output are
    NCHW tensors as torch modules exchange them; channels-last memory format makes both sides
    zero-copy views of the NHWC buffers the kernel reads and writes."""

    def __init__(self, spfilter: bw.BlockwiseSpFilter, stride: int, bias: torch.Tensor | None, info: dict | None = None):
        super().__init__()
        self.spfilter, self.stride = spfilter, int(stride)
        self.in_channels, self.out_channels, self.kernel_size = spfilter.C, spfilter.F, spfilter.R
        self.info = info or {}
        self.register_buffer("bias", None if bias is None else bias.detach().to(torch.float16))
        self._uploaded_on = None

    @classmethod
    def from_dense(cls, conv: nn.Conv2d, V: int = 64, density: float = 0.2, permute: bool = True, seed=None):
        kh, kw = conv.kernel_size
        if kh != kw or kh % 2 == 0 or conv.padding not in ((kh // 2, kh // 2), kh // 2) or conv.dilation not in ((1, 1), 1) \
                or conv.groups != 1 or conv.stride[0] != conv.stride[1] or conv.padding_mode != "zeros":
            raise ValueError("ShflBWConv2d: square odd kernel, padding = kernel // 2, equal strides, no dilation / groups")
        if conv.in_channels % 8:
            raise ValueError("ShflBWConv2d: in_channels must be a multiple of 8")
        f, info = prune_conv_filter(conv.weight.detach().float().cpu().numpy(), V, density, permute, seed=seed)
        return cls(f, conv.stride[0], conv.bias, info)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _require_cuda_half(x, "ShflBWConv2d")
        if x.dim() != 4 or x.shape[1] != self.in_channels:
            raise ValueError(f"expected [N][{self.in_channels}][H][W]")
        if self._uploaded_on != x.device:
            with torch.cuda.device(x.device):
                self.spfilter.transform_and_sync_device()
            self._uploaded_on = x.device
        n, _, h, w = x.shape
        x_nhwc = x.permute(0, 2, 3, 1).contiguous()          # a view when x is channels-last
        ho, wo = -(-h // self.stride), -(-w // self.stride)
        out = torch.empty((n, ho, wo, self.out_channels), dtype=torch.float16, device=x.device)
        with torch.cuda.device(x.device):
            op = bw.SpconvBlockwiseOp().initialize(self.spfilter, n, h, w, self.stride, x_nhwc, out)
            op(torch.cuda.current_stream(x.device))
        if self.bias is not None:
            out += self.bias.to(x.device)
        return out.permute(0, 3, 1, 2)                       # NCHW view of the NHWC result (channels-last)

    def dense_weight(self) -> torch.Tensor:
        """The pruned filter as a dense [F][C][R][S] fp16 tensor, for checks."""
        d = densify(self.spfilter).reshape(self.out_channels, self.kernel_size, self.kernel_size, self.in_channels)
        return torch.from_numpy(np.ascontiguousarray(d.transpose(0, 3, 1, 2)))


def densify(m) -> np.ndarray:
    """Logical dense matrix (rows in original order) of a Shfl-BW object, fp16."""
    d = np.zeros((m.nrow, m.ncol), np.float16)
    v = np.asarray(m.values).view(np.float16).reshape(-1, m.brow)   # one row per stored column
    perm = m.row_permute_ids if m.row_permute else np.arange(m.nrow)
    bcol = m.bcol
    indptr = m.indptr * bcol
    indices = (m.indices[:, None] * bcol + np.arange(bcol)[None, :]).reshape(-1)
    for i in range(m.nrow // m.brow):
        rows = perm[i * m.brow:(i + 1) * m.brow]
        cols = indices[indptr[i]:indptr[i + 1]]
        d[np.ix_(rows, cols)] = v[indptr[i]:indptr[i + 1]].T
    return d
