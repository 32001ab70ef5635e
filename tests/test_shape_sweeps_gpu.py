"""Parity over the benchmark sweeps' shapes (GPU, through the C ABI, against the CPU oracle).

* SpMM: transformer projection shapes M x K in {3072x768, 768x3072, 4096x4096, 11008x4096},
  row-block heights 32/64/128, densities 0.05 .. 0.5 -- the synthetic stand-ins for the
  reference's GEMM sweep list (scripts/benchmark/gemm.block_sparse.sh:8-42).  The GPU computes
  all N columns; the oracle checks a 64-column slice (columns are independent), which keeps
  the CPU side to seconds.
* SpConv: the 22 pruned layer shapes of the ResNet-50 stack as the reference's sweep encodes
  them (scripts/benchmark/conv.block_sparse.sh:5-27; H, W there are OUTPUT sizes), V=64,
  density 0.2, at a small batch.

Tolerance: |got - ref| <= max(1e-2*|ref|, 1e-3) (conftest.assert_close_fp16)."""
import numpy as np
import pytest

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import run_spconv, run_spmm

pytestmark = pytest.mark.gpu

SPMM_SHAPES = [
    # M, K, N, V, density
    (3072, 768, 512, 32, 0.05),
    (3072, 768, 512, 128, 0.5),
    (768, 3072, 512, 64, 0.25),
    (768, 3072, 4096, 128, 0.05),
    (4096, 4096, 512, 32, 0.1),
    (11008, 4096, 512, 128, 0.05),
    (11008, 4096, 512, 64, 0.1),
    (11008, 4096, 512, 32, 0.25),
]


@pytest.mark.parametrize("M,K,N,V,d", SPMM_SHAPES)
def test_spmm_sweep_shape(M, K, N, V, d):
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, d, True, 2021, values="uniform")
    B = sb.uniform_half(5000 + M + V, K * N).reshape(K, N)
    D, op = run_spmm(m, N, B)
    assert op._state.kernel == sb.KERNEL_TCGEN05
    # 64 columns spread over the token tiles: first, a middle and the last 16-column groups
    cols = np.r_[0:16, N // 2 - 8:N // 2 + 8, N - 32:N]
    perm = m.row_permute_ids if m.row_permute else None
    ref = oa.spmm_ref(M, len(cols), V, m.indptr, m.indices, m.values, perm, np.ascontiguousarray(B[:, cols]))
    assert_close_fp16(D[:, cols], ref, what=f"spmm {M}x{K}x{N} V={V} d={d}")


# (Hout, Wout, C, F, R, S, stride)
RESNET50_LAYERS = [
    (56, 56, 64, 64, 1, 1, 1), (56, 56, 256, 64, 1, 1, 1), (56, 56, 64, 64, 3, 3, 1), (56, 56, 64, 256, 1, 1, 1),
    (56, 56, 256, 128, 1, 1, 1), (28, 28, 512, 128, 1, 1, 1), (28, 28, 128, 128, 3, 3, 2), (28, 28, 128, 128, 3, 3, 1),
    (28, 28, 128, 512, 1, 1, 1), (28, 28, 256, 512, 1, 1, 2), (28, 28, 512, 256, 1, 1, 1), (14, 14, 1024, 256, 1, 1, 1),
    (14, 14, 256, 256, 3, 3, 2), (14, 14, 256, 256, 3, 3, 1), (14, 14, 256, 1024, 1, 1, 1), (14, 14, 512, 1024, 1, 1, 2),
    (14, 14, 1024, 512, 1, 1, 1), (7, 7, 2048, 512, 1, 1, 1), (7, 7, 512, 512, 3, 3, 2), (7, 7, 512, 512, 3, 3, 1),
    (7, 7, 512, 2048, 1, 1, 1), (7, 7, 1024, 2048, 1, 1, 2),
]


@pytest.mark.parametrize("Ho,Wo,Cc,F,R,S,stride", RESNET50_LAYERS)
def test_resnet50_layer_shape(Ho, Wo, Cc, F, R, S, stride):
    Bn = 3 if Ho >= 28 else 10          # not multiples of 8: the batch padding path is part of the check
    Hin, Win = Ho * stride, Wo * stride
    f = sb.BlockwiseSpFilter().init_random(F, R, S, Cc, 64, 1, 0.2, True, 2021, values="uniform")
    x = sb.uniform_half(6000 + Ho + Cc + F, Bn * Hin * Win * Cc).reshape(Bn, Hin, Win, Cc)
    O, op = run_spconv(f, Bn, Hin, Win, stride, x)
    assert op._state.kernel == sb.KERNEL_TCGEN05
    perm = f.row_permute_ids if f.row_permute else None
    ref = oa.spconv_ref_nhwc(Bn, Hin, Win, Cc, F, R, S, stride, 64, f.indptr, f.indices, f.values, perm, x)
    assert_close_fp16(O, ref, what=f"resnet layer {Ho}x{Wo} C={Cc} F={F} {R}x{S}/{stride}")
