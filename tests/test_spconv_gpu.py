"""SpConv parity on the GPU (NHWC in / NHWC out) through the C ABI, against the CPU oracle,
the committed reference fixtures (reference layouts, transposed here: pure data movement)
and the reference's own CUDA kernel.  Same tolerance as SpMM: max(1e-2*|ref|, 1e-3)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import dev, host, run_spconv

pytestmark = pytest.mark.gpu


def _arrays(f):
    return f.indptr, f.indices, f.values, (f.row_permute_ids if f.row_permute else None)


def _oracle(f, Bn, Hin, Win, stride, x, alpha=1.0):
    indptr, indices, values, perm = _arrays(f)
    return oa.spconv_ref_nhwc(Bn, Hin, Win, f.C, f.F, f.R, f.S, stride, f.brow, indptr, indices, values, perm, x, alpha)


def test_reference_fixture_outputs(golden_dir):
    z = np.load(golden_dir / "spconv_cases.npz")
    for i in range(int(z["n_cases"])):
        Bn, H, W, Cc, F, R, S, st, V, perm, seed = (int(v) for v in z[f"v{i}_args"])
        indices = z[f"v{i}_indices"]
        f = sb.BlockwiseSpFilter.from_arrays(F, R, S, Cc, V, z[f"v{i}_indptr"], indices,
                                             sb.uniform_half(seed, indices.size * V), z[f"v{i}_perm"] if perm else None)
        x_chwn = sb.uniform_half(seed + 1000, Cc * H * W * Bn).reshape(Cc, H, W, Bn)
        x = np.ascontiguousarray(x_chwn.transpose(3, 1, 2, 0))
        O, _ = run_spconv(f, Bn, H, W, st, x)
        ref = z[f"v{i}_O"].transpose(3, 1, 2, 0)[:, : O.shape[1], : O.shape[2], :]
        assert_close_fp16(O, ref, what=f"conv fixture {i}")


@pytest.mark.parametrize("V", [32, 64, 128])
@pytest.mark.parametrize("permute", [False, True])
@pytest.mark.parametrize("stride", [1, 2])
def test_3x3_small(V, permute, stride):
    Bn, H, W, Cc, F = 8, 9, 7, 32, 2 * V
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, V, 1, 0.2, permute, 5 + V, values="uniform")
    x = sb.uniform_half(77, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    O, op = run_spconv(f, Bn, H, W, stride, x)
    assert op.launches_per_exec == (3 if permute else 2)
    assert_close_fp16(O, _oracle(f, Bn, H, W, stride, x), what=f"3x3 V={V} perm={permute} stride={stride}")


@pytest.mark.parametrize("Bn", [1, 2, 5, 16, 24, 40])
def test_batch_not_multiple_of_8_and_1x1(Bn):
    f = sb.BlockwiseSpFilter().init_random(128, 1, 1, 64, 64, 1, 0.25, True, 9, values="uniform")
    x = sb.uniform_half(78 + Bn, Bn * 6 * 5 * 64).reshape(Bn, 6, 5, 64)
    O, _ = run_spconv(f, Bn, 6, 5, 1, x, alpha=0.25)
    assert_close_fp16(O, _oracle(f, Bn, 6, 5, 1, x, 0.25), what=f"1x1 batch {Bn}")


@pytest.mark.parametrize("tokens", [128, 256])
@pytest.mark.parametrize("stride", [1, 2])
def test_reference_test_shape_int9(tokens, stride):
    """The reference's conv test cases (n,h,w,c,f,r,s) = (128,14,14,256,256,3,3) at stride 1 and 2
    (test/test.spconv.blockwise.cu:10-15), d=0.1, seed 2021, integer inputs, its exact acceptance
    rule; run at batch 16 to bound CPU time, and with the filter permutation ON (the reference
    never tests that path).  Stride 2 follows the standard definition Ho = ceil(Hin / 2)."""
    ctypes.CDLL(None).srand(3)
    f = sb.BlockwiseSpFilter().init_random(256, 3, 3, 256, 64, 1, 0.1, True, 2021, values="int9")
    x = np.random.default_rng(5).integers(-4, 5, (16, 14, 14, 256)).astype(np.float16)
    O, op = run_spconv(f, 16, 14, 14, stride, x, tokens=tokens)
    assert op._state.tokens_per_cta == tokens and O.shape == (16, 14 // stride, 14 // stride, 256)
    assert oa.ref_rule_violations(O, _oracle(f, 16, 14, 14, stride, x)) == 0


def test_simt_cross_check_kernel_matches_oracle():
    f = sb.BlockwiseSpFilter().init_random(64, 3, 3, 16, 32, 1, 0.3, True, 2, values="uniform")
    x = sb.uniform_half(3, 4 * 6 * 6 * 16).reshape(4, 6, 6, 16)
    O, _ = run_spconv(f, 4, 6, 6, 2, x, kernel=sb.KERNEL_SIMT)
    assert_close_fp16(O, _oracle(f, 4, 6, 6, 2, x), what="simt conv")


def test_headline_16x14x14x512_to_2048():
    """The headline SpConv (16x14x14x512 -> 2048, 3x3, V=64, d=0.1, permuted) at full size."""
    Bn, H, W, Cc, F, V = 16, 14, 14, 512, 2048, 64
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, V, 1, 0.1, True, 2021, values="uniform")
    assert f.nnzb == 14746
    x = sb.uniform_half(8, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    O, op = run_spconv(f, Bn, H, W, 1, x)
    O2, _ = run_spconv(f, Bn, H, W, 1, x)
    assert np.array_equal(O.view(np.uint16), O2.view(np.uint16))          # deterministic
    indptr, indices, values, perm = _arrays(f)
    f_np = sb.BlockwiseSpFilter.from_arrays(F, 3, 3, Cc, V, indptr, indices, values, None)
    O_np, _ = run_spconv(f_np, Bn, H, W, 1, x)
    assert np.array_equal(O[..., perm].view(np.uint16), O_np.view(np.uint16))  # permutation = pure scatter
    assert_close_fp16(O, _oracle(f, Bn, H, W, 1, x), what="config 3 vs oracle")
    O_simt, _ = run_spconv(f, Bn, H, W, 1, x, kernel=sb.KERNEL_SIMT)
    assert_close_fp16(O, O_simt.astype(np.float32), what="config 3 vs simt")


@pytest.mark.skipif(oa.ref_gpu() is None, reason="oracle/_ref/libshflbw_ref_gpu.so (the reference's CUDA kernels) is not built")
def test_headline_against_the_reference_cuda_kernel():
    """Same shape against the reference's own kernel (its layouts: input [C][H][W][B], output [F][H][W][B])."""
    Bn, H, W, Cc, F, V = 16, 14, 14, 512, 2048, 64
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, V, 1, 0.1, True, 2021, values="uniform")
    x = sb.uniform_half(8, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    O, _ = run_spconv(f, Bn, H, W, 1, x)
    indptr, indices, values, perm = _arrays(f)
    xd = dev(np.ascontiguousarray(x.transpose(3, 1, 2, 0)))
    od = torch.zeros((F, H, W, Bn), dtype=torch.float16, device="cuda")
    cfg = oa.ref_gpu_conv_configs(V)[0][0]
    rc, _ = oa.ref_gpu_spconv(cfg, Bn, H, W, Cc, F, 3, 3, 1, V, indptr, indices, values, perm, xd.data_ptr(), od.data_ptr())
    assert rc == 0
    assert_close_fp16(O, host(od).astype(np.float32).transpose(3, 1, 2, 0), what="config 3 vs reference CUDA kernel")


def test_host_buffer_call_equals_device_call():
    f = sb.BlockwiseSpFilter().init_random(128, 3, 3, 32, 64, 1, 0.2, True, 31, values="uniform")
    x = sb.uniform_half(32, 8 * 10 * 10 * 32).reshape(8, 10, 10, 32)
    O_dev, _ = run_spconv(f, 8, 10, 10, 1, x)
    O_host = np.zeros((8, 10, 10, 128), np.float16)
    sb.spconv_host(f, 8, 10, 10, 1, x, O_host)
    assert np.array_equal(O_host.view(np.uint16), O_dev.view(np.uint16))


@pytest.mark.parametrize("tokens", [128, 256])
@pytest.mark.parametrize("permute", [False, True])
def test_filter_block_height_16_on_the_tensor_cores(permute, tokens):
    """V = 16 (the reference instantiates it, spconv/blockwise_library.cu:16-32) on the tcgen05
    kernel (one or two 128-position accumulators per item), at a ResNet-50 shape with batch 32
    (more than 65535 output positions)."""
    Bn, H, W, Cc, F = 32, 56, 56, 64, 64
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, 16, 1, 0.2, permute, 2, values="uniform")
    x = sb.uniform_half(716, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    O, op = run_spconv(f, Bn, H, W, 1, x, tokens=tokens)
    assert op._state.kernel == sb.KERNEL_TCGEN05 and op._state.tokens_per_cta == tokens
    assert_close_fp16(O, _oracle(f, Bn, H, W, 1, x), what="conv V=16")
    f2 = sb.BlockwiseSpFilter().init_random(64, 3, 3, 16, 16, 1, 0.3, True, 2, values="uniform")
    x2 = sb.uniform_half(717, 4 * 6 * 5 * 16).reshape(4, 6, 5, 16)
    O2, _ = run_spconv(f2, 4, 6, 5, 2, x2, tokens=tokens)
    assert_close_fp16(O2, _oracle(f2, 4, 6, 5, 2, x2), what="conv V=16 small, stride 2")


def test_plain_kernel_takes_more_than_65535_output_positions():
    Bn, H, W, Cc, F = 24, 56, 56, 16, 32          # 75264 positions
    f = sb.BlockwiseSpFilter().init_random(F, 1, 1, Cc, 32, 1, 0.5, True, 4, values="uniform")
    x = sb.uniform_half(718, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    O, op = run_spconv(f, Bn, H, W, 1, x, kernel=sb.KERNEL_SIMT)
    assert op._state.kernel == sb.KERNEL_SIMT
    assert_close_fp16(O, _oracle(f, Bn, H, W, 1, x), what="plain conv kernel, 75264 positions")


def test_states_stay_valid_when_a_later_init_needs_larger_scratch():
    """The filter handle owns the conv scratch; a later, larger init must not pull it from
    under a state made earlier."""
    f = sb.BlockwiseSpFilter().init_random(128, 3, 3, 32, 64, 1, 0.3, True, 12, values="uniform")
    f.transform_and_sync_device()
    x1 = sb.uniform_half(81, 2 * 5 * 5 * 32).reshape(2, 5, 5, 32)
    x2 = sb.uniform_half(82, 16 * 12 * 12 * 32).reshape(16, 12, 12, 32)
    x1d, x2d = dev(x1), dev(x2)
    o1 = torch.zeros((2, 5, 5, 128), dtype=torch.float16, device="cuda")
    o2 = torch.zeros((16, 12, 12, 128), dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream()
    op1 = sb.SpconvBlockwiseOp().initialize(f, 2, 5, 5, 1, x1d, o1)
    op1(s)
    op2 = sb.SpconvBlockwiseOp().initialize(f, 16, 12, 12, 1, x2d, o2)    # larger: scratch grows
    op2(s)
    o1.zero_()
    op1(s)                                                                 # the earlier state again
    torch.cuda.synchronize()
    f.device_status()
    assert_close_fp16(host(o1), _oracle(f, 2, 5, 5, 1, x1), what="small state after growth")
    assert_close_fp16(host(o2), _oracle(f, 16, 12, 12, 1, x2), what="large state")


def test_host_buffer_call_pipelines_large_batches_in_chunks():
    """B >= 32: the host-buffer call splits the batch into chunks of whole 8-image groups
    (here 16 + 16 + 8) whose copies and kernels overlap."""
    Bn, H, W, Cc, F = 40, 6, 5, 32, 128
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, 64, 1, 0.3, True, 19, values="uniform")
    x = sb.uniform_half(91, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    out = np.full((Bn, H, W, F), np.float16(7), np.float16)
    sb.spconv_host(f, Bn, H, W, 1, x, out, alpha=0.5)
    f.device_status()
    assert_close_fp16(out, _oracle(f, Bn, H, W, 1, x, 0.5), what="chunked host conv")


def test_both_work_item_orders_give_the_same_bits(monkeypatch):
    """SpConv decodes its work items block-major by default; the tile-major order (an override) must
    give the same output bits."""
    Bn, H, W, Cc, F, V = 8, 14, 14, 64, 256, 64
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, V, 1, 0.2, True, 9, values="uniform")
    x = sb.uniform_half(10, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    out = {}
    for order in ("0", "1"):
        monkeypatch.setenv("SHFLBW_ITEM_ORDER", order)
        out[order], _ = run_spconv(f, Bn, H, W, 1, x)
    assert_close_fp16(out["1"], _oracle(f, Bn, H, W, 1, x), what="tile-major conv")
    assert np.array_equal(out["0"].view(np.uint16), out["1"].view(np.uint16))

