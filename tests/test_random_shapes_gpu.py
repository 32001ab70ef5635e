"""Seeded random shapes through the C ABI against the CPU oracle: block heights 16/32/64/128,
V x bcol blocks, permutation on and off, ragged dense widths, alpha / beta, both token tiles,
1x1 and 3x3 filters at stride 1 and 2.  Tolerance: conftest.assert_close_fp16 (fp16 in/out, fp32
accumulate: |got - ref| <= max(1e-2*|ref|, 1e-3))."""
import numpy as np
import pytest

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import run_spconv, run_spmm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_spmm_shapes(seed):
    rng = np.random.default_rng(seed)
    for case in range(40):
        V = int(rng.choice([16, 32, 64, 128]))
        M = int(rng.integers(1, 9)) * V
        K = int(rng.integers(1, 80)) * 8
        N = int(rng.integers(1, 200)) * 8
        d = float(rng.choice([0.02, 0.1, 0.3, 0.7, 1.0]))
        bcol = int(rng.choice([1, 1, 1, 2, 4])) if K % 4 == 0 else 1
        perm = bool(rng.integers(0, 2))
        m = sb.BlockwiseSpMatrix().init_random(M, K, V, bcol, d, perm, int(rng.integers(1, 1 << 30)), values="uniform")
        B = sb.uniform_half(int(rng.integers(1, 1 << 30)), K * N).reshape(K, N)
        beta = float(rng.choice([0.0, 0.0, 1.0, -0.5]))
        alpha = float(rng.choice([1.0, 0.5, 2.0]))
        Cm = sb.uniform_half(7 + case, M * N).reshape(M, N) if beta != 0 else None
        tokens = [None, 128, 256][int(rng.integers(0, 3))]
        D, op = run_spmm(m, N, B, alpha, Cm, beta, tokens=tokens)
        if bcol > 1:
            ip, ix, v = oa.expand_block_columns(V, bcol, m.indptr, m.indices, m.values)
        else:
            ip, ix, v = m.indptr, m.indices, m.values
        ref = oa.spmm_ref(M, N, V, ip, ix, v, m.row_permute_ids if perm else None, B, alpha, Cm, beta)
        assert_close_fp16(D, ref, what=f"seed {seed} case {case}: M={M} K={K} N={N} V={V} bcol={bcol} d={d} perm={perm} "
                                       f"alpha={alpha} beta={beta} tile={op._state.tokens_per_cta} variant={op._state.variant}")


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_spconv_shapes(seed):
    rng = np.random.default_rng(seed)
    for case in range(40):
        V = int(rng.choice([16, 32, 64, 128]))
        F = int(rng.integers(1, 5)) * V
        Cc = int(rng.integers(1, 9)) * 8
        R = int(rng.choice([1, 3]))
        stride = int(rng.choice([1, 1, 2]))
        Bn, H, W = int(rng.integers(1, 20)), int(rng.integers(3, 15)), int(rng.integers(3, 15))
        d = float(rng.choice([0.05, 0.2, 0.6, 1.0]))
        perm = bool(rng.integers(0, 2))
        f = sb.BlockwiseSpFilter().init_random(F, R, R, Cc, V, 1, d, perm, int(rng.integers(1, 1 << 30)), values="uniform")
        x = sb.uniform_half(int(rng.integers(1, 1 << 30)), Bn * H * W * Cc).reshape(Bn, H, W, Cc)
        tokens = [None, 128, 256][int(rng.integers(0, 3))]
        O, op = run_spconv(f, Bn, H, W, stride, x, tokens=tokens)
        ref = oa.spconv_ref_nhwc(Bn, H, W, Cc, F, R, R, stride, V, f.indptr, f.indices, f.values,
                                 f.row_permute_ids if perm else None, x)
        assert_close_fp16(O, ref, what=f"seed {seed} case {case}: B={Bn} H={H} W={W} C={Cc} F={F} {R}x{R}/{stride} V={V} d={d} "
                                       f"perm={perm} tile={op._state.tokens_per_cta} variant={op._state.variant}")
