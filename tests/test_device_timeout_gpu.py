"""A bounded in-kernel wait that runs out: the failure path of the panel kernel.

Every barrier wait in the kernel has a limit; when it passes, the kernel records a code in the
matrix's status word, every role stops issuing work, what is in flight gets a bounded time to
land, TMEM is freed and the kernel returns.  Nothing traps, faults or hangs, and the context
stays usable.

The failure is made on purpose in a separate build of the library (-DSHFLBW_FAULT_INJECT; the
product library has no such switch): one producer warp stops arriving on the "stage is full"
barriers, so the MMA thread's wait for that stage can never complete.  With the limit lowered to
about a millisecond the launch must come back quickly, `shflbw_matrix_device_status` must report
SHFLBW_ERR_DEVICE_TIMEOUT with the code of a waiter downstream of the withheld stage, and the
next ordinary launch must give the correct result again.
"""
import ctypes as C
import time

import numpy as np
import pytest
import torch

import shflbw_sparse_nn_b200 as sb
from gpu_util import dev, host
from shflbw_sparse_nn_b200 import _cabi
from shflbw_sparse_nn_b200.build import build_fault_inject_library

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("swap", ["1", "0"])
def test_wait_limit_runs_out_and_the_library_recovers(swap, monkeypatch):
    monkeypatch.setenv("SHFLBW_SWAP", swap)      # both kernel orientations share the failure path
    flib = _cabi.load_library(build_fault_inject_library())
    flib.shflbw_debug_withhold_arrivals_from.restype = C.c_int
    flib.shflbw_debug_withhold_arrivals_from.argtypes = [C.c_int]
    M, K, N, V = 512, 512, 512, 64
    h = C.c_void_p()
    assert flib.shflbw_matrix_create_random(M, K, V, 1, 0.3, 1, 2021, _cabi.VALUES_UNIFORM, C.byref(h)) == _cabi.OK
    try:
        assert flib.shflbw_matrix_to_device(h) == _cabi.OK
        Bd = dev(sb.uniform_half(5, K * N).reshape(K, N))
        Dd = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        st = _cabi.SpmmState()
        assert flib.shflbw_spmm_init(h, N, Bd.data_ptr(), 1.0, None, 0.0, Dd.data_ptr(), _cabi.KERNEL_AUTO,
                                     C.byref(st)) == _cabi.OK
        assert st.variant == int(swap)
        stream = torch.cuda.current_stream().cuda_stream

        def launch():
            assert flib.shflbw_spmm_exec(C.byref(st), stream) == _cabi.OK
            torch.cuda.synchronize()

        launch()
        assert flib.shflbw_matrix_device_status(h) == _cabi.OK
        good = host(Dd).copy()
        assert np.abs(good.astype(np.float32)).max() > 0

        # the withheld arrival, with a limit of ~1 ms (2e6 clocks)
        assert flib.shflbw_set_wait_limit_cycles(2_000_000) == _cabi.OK
        assert flib.shflbw_debug_withhold_arrivals_from(1) == _cabi.OK
        t0 = time.perf_counter()
        launch()                                              # returns: the wait gave up
        assert time.perf_counter() - t0 < 2.0
        assert flib.shflbw_matrix_device_status(h) == _cabi.ERR_DEVICE_TIMEOUT
        # whichever waiter's limit passes first records its code: the MMA thread waiting for the
        # stage (1, TIMEOUT_FULL) or an epilogue warp waiting for the accumulator behind it (3)
        assert flib.shflbw_last_cuda_error().decode() in ("device status word = 1", "device status word = 3")
        assert flib.shflbw_matrix_device_status(h) == _cabi.OK                 # reading the word clears it

        # back to normal: same launch, correct result, clean status
        assert flib.shflbw_debug_withhold_arrivals_from(-1) == _cabi.OK
        assert flib.shflbw_set_wait_limit_cycles(400_000_000) == _cabi.OK
        Dd.zero_()
        launch()
        assert flib.shflbw_matrix_device_status(h) == _cabi.OK
        assert np.array_equal(host(Dd).view(np.uint16), good.view(np.uint16))
    finally:
        flib.shflbw_matrix_destroy(h)
