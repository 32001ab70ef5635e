"""Helpers for the GPU parity tests: device buffers through torch, calls through the C ABI."""
from __future__ import annotations

import os
from contextlib import contextmanager

import numpy as np
import torch

import shflbw_sparse_nn_b200 as sb


def dev(a: np.ndarray) -> torch.Tensor:
    """numpy fp16 array -> CUDA tensor (bit-preserving)."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.float16)


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().view(torch.int16).numpy().view(np.float16)


@contextmanager
def tile(tokens):
    """Force the tokens-per-CTA tile (128 or 256) for ops initialised inside the block."""
    old = os.environ.get("SHFLBW_TILE")
    if tokens is None:
        os.environ.pop("SHFLBW_TILE", None)
    else:
        os.environ["SHFLBW_TILE"] = str(tokens)
    try:
        yield
    finally:
        if old is None:
            os.environ.pop("SHFLBW_TILE", None)
        else:
            os.environ["SHFLBW_TILE"] = old


@contextmanager
def operand_swap(mode):
    """Force (1) or forbid (0) the rows-in-lanes kernels for ops initialised inside the block;
    None leaves the library's own choice."""
    old = os.environ.get("SHFLBW_SWAP")
    if mode is None:
        os.environ.pop("SHFLBW_SWAP", None)
    else:
        os.environ["SHFLBW_SWAP"] = str(int(mode))
    try:
        yield
    finally:
        if old is None:
            os.environ.pop("SHFLBW_SWAP", None)
        else:
            os.environ["SHFLBW_SWAP"] = old


@contextmanager
def epilogue_warps(n):
    """Force the 8- or 16-epilogue-warp kernels (tokens in lanes, 64-row blocks, 256-token tile)
    for ops initialised inside the block; None leaves the library's own choice."""
    old = os.environ.get("SHFLBW_EPILOGUE_WARPS")
    if n is None:
        os.environ.pop("SHFLBW_EPILOGUE_WARPS", None)
    else:
        os.environ["SHFLBW_EPILOGUE_WARPS"] = str(int(n))
    try:
        yield
    finally:
        if old is None:
            os.environ.pop("SHFLBW_EPILOGUE_WARPS", None)
        else:
            os.environ["SHFLBW_EPILOGUE_WARPS"] = old


def run_spmm(m, N, B, alpha=1.0, Cm=None, beta=0.0, kernel=sb.KERNEL_AUTO, tokens=None, poison=True):
    """D = alpha*A.B + beta*C on the GPU through SpmmBlockwiseOp; returns D as numpy fp16."""
    m.transform_and_sync_device()
    Bd = dev(B)
    Cd = None if Cm is None else dev(Cm)
    Dd = torch.full((m.nrow, N), float("nan") if poison else 0.0, dtype=torch.float16, device="cuda")
    with tile(tokens):
        op = sb.SpmmBlockwiseOp(kernel)
        if Cm is None and beta == 0.0 and alpha == 1.0:
            op.initialize(m, N, Bd, Dd)
        else:
            op.initialize(m, N, Bd, alpha, Cd, beta, Dd)
    op(torch.cuda.current_stream())
    torch.cuda.synchronize()
    m.device_status()
    return host(Dd), op


def run_spconv(f, Bn, Hin, Win, stride, x_nhwc, alpha=1.0, kernel=sb.KERNEL_AUTO, tokens=None):
    f.transform_and_sync_device()
    Ho, Wo = -(-Hin // stride), -(-Win // stride)
    xd = dev(x_nhwc)
    od = torch.full((Bn, Ho, Wo, f.F), float("nan"), dtype=torch.float16, device="cuda")
    with tile(tokens):
        op = sb.SpconvBlockwiseOp(kernel).initialize(f, Bn, Hin, Win, stride, xd, od, alpha)
    op(torch.cuda.current_stream())
    torch.cuda.synchronize()
    f.device_status()
    return host(od), op
