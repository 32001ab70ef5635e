"""Chained SpConv layers (activations stay channel-major, halo-padded and in stored filter order
between layers; include/shflbw.h "Chained SpConv layers"): GPU parity against the unchained
path and the CPU oracle.  A single chained layer performs exactly the arithmetic of the
unchained one, so it must match bit for bit; a second layer sums its folded (re-sorted)
columns in another order, so it is held to |got - ref| <= max(1e-2*|ref|, 1e-3)."""
import numpy as np
import pytest
import torch

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import dev, epilogue_warps, host, operand_swap, run_spconv, tile

pytestmark = pytest.mark.gpu


def _chain_buf(C_, H, W, B, R, S):
    return torch.zeros(sb.chain_buffer_elems(C_, H, W, B, R, S), dtype=torch.float16, device="cuda")


@pytest.mark.parametrize("V,Bn,relu,swap", [(32, 8, False, None), (64, 3, True, 0), (64, 3, True, 1), (128, 16, True, 0),
                                             (128, 16, False, 1)])
def test_one_chained_layer_equals_the_unchained_layer_bit_for_bit(V, Bn, relu, swap):
    H, W, Cc, F = 9, 7, 32, 2 * V
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, V, 1, 0.25, True, 11 + V, values="uniform")
    x = sb.uniform_half(500 + V, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    ref, _ = run_spconv(f, Bn, H, W, 1, x)                      # NHWC, inverse permutation applied
    if relu:
        ref = np.maximum(ref, np.float16(0))
    xd = dev(x)
    b0, b1 = _chain_buf(Cc, H, W, Bn, 3, 3), _chain_buf(F, H, W, Bn, 1, 1)
    y = torch.full((Bn, H, W, F), float("nan"), dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream()
    sb.chain_import_nhwc(xd, Bn, H, W, Cc, 3, 3, b0, s)
    with operand_swap(swap):          # both kernel orientations (rows or tokens in TMEM lanes)
        op = sb.SpconvChainOp().initialize(f, Bn, H, W, 1, b0, b1, 1, 1, relu=relu)
    assert op.launches_per_exec == 1 and (swap is None or op._state.variant == swap)
    for _ in range(2):                                          # buffers are reusable without re-zeroing
        op(s)
    sb.chain_export_nhwc(b1, Bn, H, W, F, 1, 1, f, y, s)
    torch.cuda.synchronize()
    f.device_status()
    got = host(y)
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("stride2", [1, 2])
def test_two_chained_layers_match_oracle_and_unchained_path(stride2):
    Bn, H, W, C0, F1, F2, V = 5, 12, 10, 32, 128, 64, 32
    f1 = sb.BlockwiseSpFilter().init_random(F1, 3, 3, C0, V, 1, 0.3, True, 21, values="uniform")
    f2 = sb.BlockwiseSpFilter().init_random(F2, 3, 3, F1, V, 1, 0.2, True, 22, values="uniform")
    f2c = f2.fold_input_order(f1)
    x = sb.uniform_half(77, Bn * H * W * C0).reshape(Bn, H, W, C0)
    # unchained: layer 1 (GPU, NHWC) -> ReLU -> layer 2 on the CPU oracle and on the GPU
    y1, _ = run_spconv(f1, Bn, H, W, 1, x, alpha=0.25)
    y1 = np.maximum(y1, np.float16(0))
    H2, W2 = -(-H // stride2), -(-W // stride2)
    ref = oa.spconv_ref_nhwc(Bn, H, W, F1, F2, 3, 3, stride2, V, f2.indptr, f2.indices, f2.values,
                             f2.row_permute_ids, y1)
    y2_unchained, _ = run_spconv(f2, Bn, H, W, stride2, y1)
    # chained
    f2c.transform_and_sync_device()
    s = torch.cuda.current_stream()
    b0, b1, b2 = _chain_buf(C0, H, W, Bn, 3, 3), _chain_buf(F1, H, W, Bn, 3, 3), _chain_buf(F2, H2, W2, Bn, 1, 1)
    y = torch.full((Bn, H2, W2, F2), float("nan"), dtype=torch.float16, device="cuda")
    sb.chain_import_nhwc(dev(x), Bn, H, W, C0, 3, 3, b0, s)
    l1 = sb.SpconvChainOp().initialize(f1, Bn, H, W, 1, b0, b1, 3, 3, alpha=0.25, relu=True)
    l2 = sb.SpconvChainOp().initialize(f2c, Bn, H, W, stride2, b1, b2, 1, 1)
    l1(s); l2(s)
    sb.chain_export_nhwc(b2, Bn, H2, W2, F2, 1, 1, f2c, y, s)
    torch.cuda.synchronize()
    f1.device_status(); f2c.device_status()
    got = host(y)
    assert_close_fp16(got, ref, what=f"chained 2 layers (stride {stride2}) vs oracle")
    assert_close_fp16(got, y2_unchained.astype(np.float32), what="chained vs unchained GPU path")


@pytest.mark.parametrize("swap", [0, 1, 2])
def test_residual_add_across_two_chained_layers(swap):
    """y = relu(conv2(relu(conv1(x))) + x): an identity shortcut around two chained layers.  x is
    imported in logical channel order, conv2's output is in conv2's stored filter order, so the
    residual planes are picked through the map of shflbw_chain_residual_map."""
    Bn, H, W, Cc, V = 6, 9, 8, 64, 64
    f1 = sb.BlockwiseSpFilter().init_random(128, 1, 1, Cc, V, 1, 0.5, True, 41, values="uniform")
    f2 = sb.BlockwiseSpFilter().init_random(Cc, 3, 3, 128, V, 1, 0.25, True, 42, values="uniform")
    f2c = f2.fold_input_order(f1)
    x = sb.uniform_half(43, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    # unchained reference on the GPU path + numpy for the elementwise part
    y1, _ = run_spconv(f1, Bn, H, W, 1, x, alpha=0.25)
    y1 = np.maximum(y1, np.float16(0))
    y2, _ = run_spconv(f2, Bn, H, W, 1, y1, alpha=0.25)
    want = np.maximum((y2 + x).astype(np.float16), np.float16(0))
    want_oracle = np.maximum(oa.spconv_ref_nhwc(Bn, H, W, 128, Cc, 3, 3, 1, V, f2.indptr, f2.indices, f2.values,
                                                f2.row_permute_ids, y1, 0.25).astype(np.float32)
                             + x.astype(np.float32), 0)
    s = torch.cuda.current_stream()
    f2c.transform_and_sync_device()
    b0 = _chain_buf(Cc, H, W, Bn, 1, 1)           # x for conv1 (1x1: no halo) -- also the residual (same geometry as y)
    b1 = _chain_buf(128, H, W, Bn, 3, 3)
    b2 = _chain_buf(Cc, H, W, Bn, 1, 1)
    y = torch.full((Bn, H, W, Cc), float("nan"), dtype=torch.float16, device="cuda")
    sb.chain_import_nhwc(dev(x), Bn, H, W, Cc, 1, 1, b0, s)
    # swap 2: tokens in lanes with sixteen epilogue warps (the kernel the library picks for shallow layers with many items)
    with operand_swap(1 if swap == 1 else 0), epilogue_warps(16 if swap == 2 else 8), tile(256 if swap == 2 else None):
        l1 = sb.SpconvChainOp().initialize(f1, Bn, H, W, 1, b0, b1, 3, 3, alpha=0.25, relu=True)
        l2 = sb.SpconvChainOp().initialize(f2c, Bn, H, W, 1, b1, b2, 1, 1, alpha=0.25, relu=True)
    assert l1._state.variant == swap and l2._state.variant == swap
    l2.set_residual(b0, residual_producer=None)    # b0 holds logical channel order
    l1(s); l2(s)
    sb.chain_export_nhwc(b2, Bn, H, W, Cc, 1, 1, f2c, y, s)
    torch.cuda.synchronize()
    f1.device_status(); f2c.device_status()
    got = host(y)
    assert_close_fp16(got, want_oracle, what=f"residual block vs oracle (swap {swap})")
    assert_close_fp16(got, want.astype(np.float32), what=f"residual block vs unchained GPU path (swap {swap})")
