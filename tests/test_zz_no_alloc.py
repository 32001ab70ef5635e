"""The SpConv entry point that never allocates (shflbw_spconv_exec_static_scratch).

It exists for callers that run where device allocation is not allowed -- a plugin's execute
hook, a serving loop whose memory was handed out up front -- and keeps its scratch in a fixed
array inside the library.  The test calls it through the C
ABI twice in a row (the array is shared and keeps the previous call's contents, so the second
call must not be disturbed by the first) and compares each result with the regular
SpconvBlockwiseOp path on the same inputs.  Both paths run the same kernels, so the results
are expected bit-identical; the assertion still uses the suite's floating-point bar
(|got - ref| <= max(1e-2*|ref|, 1e-3)).  The first call is also checked against the CPU oracle,
and the free device memory reported by the driver must be the same before and after the calls:
that is the property the entry point exists for.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import dev, host, run_spconv
from shflbw_sparse_nn_b200 import _cabi

pytestmark = pytest.mark.gpu


def _call_static(f, Bn, Hin, Win, stride, xd, od, alpha=1.0):
    """One call on buffers the caller made beforehand; returns (status, free bytes before, after)."""
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    rc = _cabi.lib().shflbw_spconv_exec_static_scratch(f._h, Bn, Hin, Win, stride, xd.data_ptr(), od.data_ptr(),
                                                       alpha, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    return rc, free0, free1


@pytest.mark.parametrize("permute", [True, False])
def test_static_scratch_matches_regular_path_twice(permute):
    Bn, H, W, Cc, F, V = 16, 14, 14, 64, 256, 64
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, V, 1, 0.2, permute, 41, values="uniform")
    f.transform_and_sync_device()
    x1 = sb.uniform_half(51, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    x2 = sb.uniform_half(52, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    ref1, _ = run_spconv(f, Bn, H, W, 1, x1, alpha=0.5)
    ref2, _ = run_spconv(f, Bn, H, W, 1, x2, alpha=0.5)
    # Every buffer exists before the calls, so any change in free memory is the library's doing.
    xd1, xd2 = dev(x1), dev(x2)
    od1 = torch.full((Bn, H, W, F), float("nan"), dtype=torch.float16, device="cuda")
    od2 = torch.full((Bn, H, W, F), float("nan"), dtype=torch.float16, device="cuda")
    _call_static(f, Bn, H, W, 1, xd1, od1, alpha=0.5)            # first call on the device: address look-up
    od1.fill_(float("nan"))
    rc1, free_a, free_b = _call_static(f, Bn, H, W, 1, xd1, od1, alpha=0.5)
    rc2, free_c, free_d = _call_static(f, Bn, H, W, 1, xd2, od2, alpha=0.5)   # reuses the same array
    assert rc1 == _cabi.OK and rc2 == _cabi.OK
    assert free_a == free_b == free_c == free_d, "the no-allocation entry point changed free device memory"
    f.device_status()
    got1, got2 = host(od1), host(od2)
    assert_close_fp16(got1, ref1.astype(np.float32), what="static scratch, call 1")
    assert_close_fp16(got2, ref2.astype(np.float32), what="static scratch, call 2")
    assert np.array_equal(got1.view(np.uint16), ref1.view(np.uint16))
    assert np.array_equal(got2.view(np.uint16), ref2.view(np.uint16))
    want = 0.5 * oa.spconv_ref_nhwc(Bn, H, W, Cc, F, 3, 3, 1, V, f.indptr, f.indices, f.values,
                                    f.row_permute_ids if permute else None, x1)
    assert_close_fp16(got1, want, what="static scratch vs CPU oracle")


def test_static_scratch_applies_the_32_bit_output_guard():
    """With an unpermuted filter the output bypasses the array, so its capacity does not bound the
    output extent; the entry point must refuse what shflbw_spconv_init refuses: B*Ho*Wo*F >= 2^32 - 1."""
    f = sb.BlockwiseSpFilter().init_random(2048, 1, 1, 8, 64, 1, 0.5, False, 3, values="uniform")
    f.transform_and_sync_device()
    Bn, H, W = 8, 512, 512
    # the staged input (2*8*512*512*8 bytes = 32 MiB) just fits the array; the output would be 2^32 elements
    assert 2 * 8 * H * W * Bn <= _cabi.STATIC_SCRATCH_BYTES and Bn * H * W * 2048 >= 2 ** 32 - 1
    tiny = torch.zeros(64, dtype=torch.float16, device="cuda")   # never dereferenced: the call is refused first
    rc = _cabi.lib().shflbw_spconv_exec_static_scratch(f._h, Bn, H, W, 1, tiny.data_ptr(), tiny.data_ptr(), 1.0, None)
    torch.cuda.synchronize()
    assert rc == _cabi.ERR_UNSUPPORTED
    st = _cabi.SpconvState()
    rc = _cabi.lib().shflbw_spconv_init(f._h, Bn, H, W, 1, tiny.data_ptr(), tiny.data_ptr(), 1.0, sb.KERNEL_AUTO, C.byref(st))
    assert rc == _cabi.ERR_UNSUPPORTED


def test_static_scratch_rejects_shapes_beyond_capacity():
    f = sb.BlockwiseSpFilter().init_random(256, 3, 3, 64, 64, 1, 0.2, True, 41, values="uniform")
    f.transform_and_sync_device()
    Bn, H, W = 64, 56, 56   # staged input alone: 2*64*56*56*64 = 25.7 MB, staged output 102.8 MB
    need = 2 * 64 * H * W * Bn + 2 * Bn * H * W * 256
    assert need > _cabi.STATIC_SCRATCH_BYTES
    x = torch.zeros((Bn, H, W, 64), dtype=torch.float16, device="cuda")
    o = torch.full((Bn, H, W, 256), 7.0, dtype=torch.float16, device="cuda")
    rc = _cabi.lib().shflbw_spconv_exec_static_scratch(f._h, Bn, H, W, 1, x.data_ptr(), o.data_ptr(), 1.0, None)
    torch.cuda.synchronize()
    assert rc == _cabi.ERR_TOO_LARGE
    assert "static scratch" in _cabi.lib().shflbw_last_cuda_error().decode()
    assert bool((o == 7.0).all())   # nothing was launched
