"""SpMM parity on the GPU, through the C ABI, against the CPU oracle, the committed
reference fixtures and the reference's own CUDA kernels (when oracle/_ref is present).

Tolerance: fp16 inputs/outputs with fp32 accumulation -> |got - ref| <= max(1e-2*|ref|, 1e-3)
(conftest.assert_close_fp16).  Integer-valued inputs use the reference's own rule
|ref - d| <= 1e-3*|ref| with no floor, which then means exact."""
import ctypes

import numpy as np
import pytest
import torch

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import dev, epilogue_warps, host, operand_swap, run_spmm

pytestmark = pytest.mark.gpu


def _arrays(m):
    return m.indptr, m.indices, m.values, (m.row_permute_ids if m.row_permute else None)


def _oracle(m, N, B, alpha=1.0, Cm=None, beta=0.0):
    indptr, indices, values, perm = _arrays(m)
    return oa.spmm_ref(m.nrow, N, m.brow, indptr, indices, values, perm, B, alpha, Cm, beta)


def test_config1_256cubed_v32_uniform():
    """The small correctness case: M=K=N=256, V=32, d=0.1, permuted, uniform[-1,1] values."""
    m = sb.BlockwiseSpMatrix().init_random(256, 256, 32, 1, 0.1, True, 2021, values="uniform")
    assert m.nnzb == 205
    B = sb.uniform_half(3021, 256 * 256).reshape(256, 256)
    D, op = run_spmm(m, 256, B)
    assert op._state.kernel == sb.KERNEL_TCGEN05
    assert_close_fp16(D, _oracle(m, 256, B), what="config 1")


def test_config1_int9_reference_rule():
    ctypes.CDLL(None).srand(1)
    m = sb.BlockwiseSpMatrix().init_random(256, 256, 32, 1, 0.1, True, 2021, values="int9")
    rng = np.random.default_rng(1)
    B = rng.integers(-4, 5, (256, 256)).astype(np.float16)
    D, _ = run_spmm(m, 256, B)
    assert oa.ref_rule_violations(D, _oracle(m, 256, B)) == 0


def test_reference_fixture_outputs(golden_dir):
    """Outputs of the reference's own get_host_reference, committed under tests/golden."""
    z = np.load(golden_dir / "spmm_cases.npz")
    for i in range(int(z["n_cases"])):
        M, K, N, V, perm, seed = (int(v) for v in z[f"s{i}_args"])
        if V not in (32, 64, 128):
            continue
        beta = float(z[f"s{i}_beta"])
        indices = z[f"s{i}_indices"]
        m = sb.BlockwiseSpMatrix.from_arrays(M, K, V, z[f"s{i}_indptr"], indices, sb.uniform_half(seed, indices.size * V),
                                             z[f"s{i}_perm"] if perm else None)
        B = sb.uniform_half(seed + 1000, K * N).reshape(K, N)
        Cm = sb.uniform_half(seed + 2000, M * N).reshape(M, N) if beta else None
        D, _ = run_spmm(m, N, B, 1.0, Cm, beta)
        assert_close_fp16(D, z[f"s{i}_D"], what=f"fixture {i}")


@pytest.mark.parametrize("V", [32, 64, 128])
@pytest.mark.parametrize("permute", [False, True])
@pytest.mark.parametrize("tokens", [128, 256])
def test_reference_test_shape_1024x960x1024(V, permute, tokens):
    """The reference's own test case (m,n,k,d,seed) = (1024,960,1024,0.1,2021), integer inputs,
    its acceptance rule; N = 960 exercises the dense-dimension residue."""
    ctypes.CDLL(None).srand(V + permute)
    m = sb.BlockwiseSpMatrix().init_random(1024, 1024, V, 1, 0.1, permute, 2021, values="int9")
    B = np.random.default_rng(V).integers(-4, 5, (1024, 960)).astype(np.float16)
    D, op = run_spmm(m, 960, B, tokens=tokens)
    assert op._state.tokens_per_cta == tokens
    assert oa.ref_rule_violations(D, _oracle(m, 960, B)) == 0


@pytest.mark.parametrize("V", [32, 64, 128])
@pytest.mark.parametrize("N", [8, 40, 136, 264, 520])
def test_dense_residue_and_alpha_beta(V, N):
    m = sb.BlockwiseSpMatrix().init_random(2 * V, 320, V, 1, 0.3, True, 11 + N, values="uniform")
    B = sb.uniform_half(50 + N, 320 * N).reshape(320, N)
    Cm = sb.uniform_half(60 + N, 2 * V * N).reshape(2 * V, N)
    D, _ = run_spmm(m, N, B, 0.5, Cm, 2.0)
    assert_close_fp16(D, _oracle(m, N, B, 0.5, Cm, 2.0), what=f"V={V} N={N} alpha/beta")
    D1, _ = run_spmm(m, N, B)
    assert_close_fp16(D1, _oracle(m, N, B), what=f"V={V} N={N}")


@pytest.mark.parametrize("V", [32, 64, 128])
def test_ragged_and_empty_row_blocks(V):
    """Column counts 0, 1, 15, 16, 17, 63, 64, 65, 130 per row block: every K-tail case."""
    counts = [0, 1, 15, 16, 17, 63, 64, 65, 130]
    K = 160
    rng = np.random.default_rng(V)
    indptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    indices = np.concatenate([np.sort(rng.choice(K, c, replace=False)) for c in counts]).astype(np.int32)
    M = V * len(counts)
    vals = sb.uniform_half(V, indices.size * V)
    perm = rng.permutation(M).astype(np.int32)
    m = sb.BlockwiseSpMatrix.from_arrays(M, K, V, indptr, indices, vals, perm)
    B = sb.uniform_half(99, K * 72).reshape(K, 72)
    D, _ = run_spmm(m, 72, B)
    ref = _oracle(m, 72, B)
    assert_close_fp16(D, ref, what=f"ragged V={V}")
    assert np.all(D[perm[:V]] == 0)  # the empty row block writes zeros, not garbage


def test_simt_cross_check_kernel_matches_oracle():
    m = sb.BlockwiseSpMatrix().init_random(256, 256, 64, 1, 0.2, True, 3, values="uniform")
    B = sb.uniform_half(4, 256 * 96).reshape(256, 96)
    D, op = run_spmm(m, 96, B, kernel=sb.KERNEL_SIMT)
    assert op._state.kernel == sb.KERNEL_SIMT
    assert_close_fp16(D, _oracle(m, 96, B), what="simt")


def test_headline_4096cubed_v64_d01():
    """The headline SpMM (4096^3, V=64, d=0.1, permuted) at full size: permutation/index handling checked exactly through
    size-independent properties, values against the oracle on a column slice and against the
    plain CUDA-core kernel on the whole matrix."""
    M = K = N = 4096
    V = 64
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, 0.1, True, 2021, values="uniform")
    assert m.nnzb == 26214
    B = sb.uniform_half(7, K * N).reshape(K, N)
    D, op = run_spmm(m, N, B)
    assert op.launches_per_exec == 1
    # (a) determinism: bitwise equal on a second run
    D2, _ = run_spmm(m, N, B)
    assert np.array_equal(D.view(np.uint16), D2.view(np.uint16))
    # (b) the inverse permutation is a pure row scatter: same matrix without permutation
    #     gives bitwise the same rows at the stored positions
    indptr, indices, values, perm = _arrays(m)
    m_np = sb.BlockwiseSpMatrix.from_arrays(M, K, V, indptr, indices, values, None)
    D_np, _ = run_spmm(m_np, N, B)
    assert np.array_equal(D[perm].view(np.uint16), D_np.view(np.uint16))
    # (c) oracle on a 64-column slice (columns are independent)
    cols = slice(1000, 1064)
    ref = oa.spmm_ref(M, 64, V, indptr, indices, values, perm, np.ascontiguousarray(B[:, cols]))
    assert_close_fp16(D[:, cols], ref, what="4096^3 slice vs oracle")
    # (d) whole matrix vs the plain CUDA-core kernel
    D_simt, _ = run_spmm(m, N, B, kernel=sb.KERNEL_SIMT)
    assert_close_fp16(D, D_simt.astype(np.float32), what="4096^3 vs simt")


@pytest.mark.skipif(oa.ref_gpu() is None, reason="oracle/_ref/libshflbw_ref_gpu.so (the reference's CUDA kernels) is not built")
def test_headline_4096cubed_against_the_reference_cuda_kernel():
    """The whole 4096 x 4096 output against the reference's own CUDA kernel on identical arrays."""
    M = K = N = 4096
    V = 64
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, 0.1, True, 2021, values="uniform")
    B = sb.uniform_half(7, K * N).reshape(K, N)
    D, _ = run_spmm(m, N, B)
    indptr, indices, values, perm = _arrays(m)
    Bd = dev(B)
    Dd = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    cfg = oa.ref_gpu_spmm_configs(V)[1][0]
    rc, _ = oa.ref_gpu_spmm(cfg, M, K, N, V, indptr, indices, values, perm, Bd.data_ptr(), Dd.data_ptr())
    assert rc == 0
    assert_close_fp16(D, host(Dd).astype(np.float32), what="4096^3 vs reference CUDA kernel")


def test_host_buffer_call_equals_device_call():
    m = sb.BlockwiseSpMatrix().init_random(512, 384, 64, 1, 0.15, True, 21, values="uniform")
    B = sb.uniform_half(22, 384 * 200).reshape(384, 200)
    D_dev, _ = run_spmm(m, 200, B)
    D_host = np.zeros((512, 200), np.float16)
    sb.spmm_host(m, 200, B, D_host)
    assert np.array_equal(D_host.view(np.uint16), D_dev.view(np.uint16))


@pytest.mark.skipif(oa.ref_host() is None, reason="oracle/_ref not present")
def test_meta_image_equals_reference_transform_and_sync_device():
    r = oa.RefMatrix.init_random(512, 384, 32, 0.15, True, 17)
    m = sb.BlockwiseSpMatrix.from_arrays(512, 384, 32, r.indptr, r.indices, r.values, r.perm)
    assert np.array_equal(m.meta_h, r.meta_image())


@pytest.mark.parametrize("tokens", [128, 256])
@pytest.mark.parametrize("permute", [False, True])
def test_row_block_height_16_reference_shape_on_the_tensor_cores(permute, tokens):
    """V = 16 (instantiated by the reference, spmm/blockwise_library.cu:15-31) runs on the tcgen05
    kernel (UMMA M = 128 tokens, N = 16; one or two accumulators per item): the reference's own
    test case (m,n,k,d,seed) = (1024,960,1024,0.1,2021), integer inputs, its exact acceptance rule
    (test/test.spmm.blockwise.cu:10-14, test_util.spmm.h:18)."""
    ctypes.CDLL(None).srand(16 + permute)
    m = sb.BlockwiseSpMatrix().init_random(1024, 1024, 16, 1, 0.1, permute, 2021, values="int9")
    B = np.random.default_rng(16).integers(-4, 5, (1024, 960)).astype(np.float16)
    D, op = run_spmm(m, 960, B, tokens=tokens)
    assert op._state.kernel == sb.KERNEL_TCGEN05 and op._state.tokens_per_cta == tokens
    assert oa.ref_rule_violations(D, _oracle(m, 960, B)) == 0


@pytest.mark.parametrize("N", [8, 136, 520])
def test_row_block_height_16_residue_alpha_beta_and_large_row_counts(N):
    """V = 16 with uniform data, a ragged dense width, alpha / beta, and more than 65535 rows."""
    m = sb.BlockwiseSpMatrix().init_random(256, 384, 16, 1, 0.2, True, 2021, values="uniform")
    B = sb.uniform_half(616, 384 * N).reshape(384, N)
    Cm = sb.uniform_half(617, 256 * N).reshape(256, N)
    D, op = run_spmm(m, N, B, 0.5, Cm, 2.0)
    assert op._state.kernel == sb.KERNEL_TCGEN05
    assert_close_fp16(D, _oracle(m, N, B, 0.5, Cm, 2.0), what=f"V=16 N={N}")
    if N == 8:   # many rows: 70000 > 65535 on both kernels (the plain kernel indexes rows in grid.x)
        big = sb.BlockwiseSpMatrix().init_random(70000 // 16 * 16, 64, 16, 1, 0.25, True, 5, values="uniform")
        Bb = sb.uniform_half(6, 64 * 8).reshape(64, 8)
        D1, _ = run_spmm(big, 8, Bb)
        D2, op2 = run_spmm(big, 8, Bb, kernel=sb.KERNEL_SIMT)
        assert op2._state.kernel == sb.KERNEL_SIMT
        assert_close_fp16(D1, _oracle(big, 8, Bb), what="V=16, 70000 rows")
        assert_close_fp16(D2, D1.astype(np.float32), what="plain kernel, 70000 rows")


@pytest.mark.parametrize("V", [64, 128])
@pytest.mark.parametrize("swap", [0, 1])
@pytest.mark.parametrize("tokens", [128, 256])
def test_both_operand_orientations(V, swap, tokens):
    """V = 64 / 128 have two kernels: tokens in TMEM lanes (UMMA M = 128 tokens, N = V) and rows in
    TMEM lanes (M = V, N = the token tile).  Both must match the oracle, with a ragged dense width,
    empty and short row blocks, alpha and beta."""
    M, K, N = 4 * V, 640, 1000
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, 0.35, True, 900 + V, values="uniform")
    B = sb.uniform_half(901, K * N).reshape(K, N)
    Cm = sb.uniform_half(902, M * N).reshape(M, N)
    with operand_swap(swap):
        D, op = run_spmm(m, N, B, alpha=0.5, Cm=Cm, beta=-1.5, tokens=tokens)
        D2, op2 = run_spmm(m, N, B, tokens=tokens)
    assert op._state.variant == swap and op2._state.variant == swap
    assert_close_fp16(D, _oracle(m, N, B, 0.5, Cm, -1.5), what=f"V={V} swap={swap} alpha/beta")
    assert_close_fp16(D2, _oracle(m, N, B), what=f"V={V} swap={swap}")


@pytest.mark.parametrize("density,N", [(0.05, 1000), (0.09, 4096), (0.35, 520)])
def test_sixteen_epilogue_warp_kernel(density, N):
    """Tokens in lanes with sixteen epilogue warps (four accumulator sets, 32-column stages, three
    producer groups): picked by the library for shallow blocks with many items, forced here also
    on deeper ones (several stages per item).  alpha, beta * C, permutation, ragged dense width,
    empty blocks."""
    M, K, V = 512, 640, 64
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, density, True, 31, values="uniform")
    B = sb.uniform_half(32, K * N).reshape(K, N)
    Cm = sb.uniform_half(33, M * N).reshape(M, N)
    with operand_swap(0), epilogue_warps(16):
        D, op = run_spmm(m, N, B, alpha=0.5, Cm=Cm, beta=-1.5, tokens=256)
        D2, op2 = run_spmm(m, N, B, tokens=256)
    assert op._state.variant == 2 and op2._state.variant == 2 and op._state.producer_warps == 3
    assert_close_fp16(D, _oracle(m, N, B, 0.5, Cm, -1.5), what="16 epilogue warps, alpha/beta")
    assert_close_fp16(D2, _oracle(m, N, B), what="16 epilogue warps")
    with operand_swap(0), epilogue_warps(8):
        D3, op3 = run_spmm(m, N, B, tokens=256)
    assert op3._state.variant == 0
    assert np.array_equal(D2.view(np.uint16), D3.view(np.uint16))    # same arithmetic, same order


def test_library_picks_sixteen_epilogue_warps_for_shallow_blocks_with_many_items():
    m = sb.BlockwiseSpMatrix().init_random(256, 256, 64, 1, 0.2, True, 5, values="uniform")   # ~51 columns per block
    N = 256 * 148
    B = sb.uniform_half(6, 256 * N).reshape(256, N)
    D, op = run_spmm(m, N, B)
    assert op._state.variant == 2
    assert_close_fp16(D, _oracle(m, N, B), what="auto 16 epilogue warps")


@pytest.mark.parametrize("N", [8, 40, 136])
def test_rows_in_lanes_kernel_with_narrow_dense_operands(N):
    """Forced rows-in-lanes kernel where the dense width is a fraction of one token tile."""
    m = sb.BlockwiseSpMatrix().init_random(128, 256, 64, 1, 0.5, True, 77, values="uniform")
    B = sb.uniform_half(78 + N, 256 * N).reshape(256, N)
    with operand_swap(1):
        D, op = run_spmm(m, N, B)
    assert op._state.variant == 1
    assert_close_fp16(D, _oracle(m, N, B), what=f"rows in lanes, N={N}")


def test_host_buffer_call_pipelines_wide_operands_in_column_chunks():
    """N >= 2048: the host-buffer call cuts the dense operand into column chunks (copy in, kernel
    and copy out overlap); ragged last chunk, alpha and beta * C included."""
    M, K, N = 256, 320, 2056                      # chunks of 768, 768 and 520 columns
    m = sb.BlockwiseSpMatrix().init_random(M, K, 64, 1, 0.3, True, 31, values="uniform")
    B = sb.uniform_half(32, K * N).reshape(K, N)
    Cm = sb.uniform_half(33, M * N).reshape(M, N)
    D_host = np.full((M, N), np.float16(7), np.float16)
    sb.spmm_host(m, N, B, D_host, alpha=0.5, C_host=Cm, beta=2.0)
    m.device_status()
    assert_close_fp16(D_host, _oracle(m, N, B, 0.5, Cm, 2.0), what="chunked host call")
    D_dev, _ = run_spmm(m, N, B, alpha=0.5, Cm=Cm, beta=2.0)
    # same kernels on the same columns: only the summation order of a token tile's partners differs -> none
    assert_close_fp16(D_host, D_dev.astype(np.float32), what="chunked host call vs device call")


@pytest.mark.parametrize("N", [1000, 264, 64])
def test_tma_tile_gather_kernel(N, monkeypatch):
    """The SpMM kernel whose producers fetch the rows of B with TMA tile::gather4 (the default for
    64-row blocks once every SM has a few 256-token items; forced here on small shapes): ragged
    dense width (the copy engine zero-fills past N), empty and short row blocks, alpha, and
    beta * C; bit-identical to the cp.async kernel, which sums in the same order."""
    monkeypatch.setenv("SHFLBW_SWAP", "1")
    M, K, V = 256, 640, 64
    counts = [0, 1, 130, 47]
    rng = np.random.default_rng(N)
    indptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    indices = np.concatenate([np.sort(rng.choice(K, c, replace=False)) for c in counts]).astype(np.int32)
    m = sb.BlockwiseSpMatrix.from_arrays(M, K, V, indptr, indices, sb.uniform_half(3, indices.size * V),
                                         rng.permutation(M).astype(np.int32))
    B = sb.uniform_half(901 + N, K * N).reshape(K, N)
    Cm = sb.uniform_half(902, M * N).reshape(M, N)
    monkeypatch.setenv("SHFLBW_GATHER", "1")
    D1, op1 = run_spmm(m, N, B, tokens=256)
    D2, op2 = run_spmm(m, N, B, alpha=0.5, Cm=Cm, beta=-1.5, tokens=256)
    assert op1._state.gather == 1 and op2._state.gather == 1 and op1._state.variant == 1
    monkeypatch.setenv("SHFLBW_GATHER", "0")
    E1, op3 = run_spmm(m, N, B, tokens=256)
    E2, _ = run_spmm(m, N, B, alpha=0.5, Cm=Cm, beta=-1.5, tokens=256)
    assert op3._state.gather == 0
    assert_close_fp16(D1, _oracle(m, N, B), what=f"TMA gather N={N}")
    assert_close_fp16(D2, _oracle(m, N, B, 0.5, Cm, -1.5), what=f"TMA gather N={N} alpha/beta")
    assert np.array_equal(D1.view(np.uint16), E1.view(np.uint16)) and np.array_equal(D2.view(np.uint16), E2.view(np.uint16))


@pytest.mark.parametrize("V,swap", [(64, 1), (64, 0), (128, 1), (32, 0)])
def test_both_work_item_orders_give_the_same_bits(V, swap, monkeypatch):
    """Work items are decoded block-major (item = block * tiles + tile) or tile-major (item = tile *
    blocks + block, the SpMM default: concurrent CTAs share a few token tiles of B).  Every item is
    computed by one CTA in the same order of additions either way, so the outputs are identical."""
    M, K, N = 6 * V, 512, 1160
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, 0.3, True, 61 + V, values="uniform")
    B = sb.uniform_half(62, K * N).reshape(K, N)
    out = {}
    for order in ("0", "1"):
        monkeypatch.setenv("SHFLBW_ITEM_ORDER", order)
        with operand_swap(swap):
            out[order], _ = run_spmm(m, N, B, alpha=0.5)
    assert_close_fp16(out["1"], _oracle(m, N, B, 0.5), what=f"tile-major V={V}")
    assert np.array_equal(out["0"].view(np.uint16), out["1"].view(np.uint16))

