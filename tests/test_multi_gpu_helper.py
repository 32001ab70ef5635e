"""The C-ABI helpers for driving several GPUs from one process (shflbw_shard_range,
shflbw_matrix_clone, shflbw_multi_*): the sparse operand is replicated on every listed device,
each device owns a contiguous slice of the dense columns (SpMM) or of the batch (SpConv), and no
exchange is needed to compute.  On a box with one GPU the same device is listed twice, which
exercises the same code (two replicas, two streams); with more GPUs the first two are used."""
import ctypes as C

import numpy as np
import pytest

import shflbw_sparse_nn_b200 as sb
from shflbw_sparse_nn_b200 import _cabi
from shflbw_sparse_nn_b200.sharding import shard_range


def _c_range(total, granule, parts, index):
    b, n = C.c_longlong(), C.c_longlong()
    rc = _cabi.lib().shflbw_shard_range(total, granule, parts, index, C.byref(b), C.byref(n))
    return rc, b.value, n.value


def test_shard_range_matches_the_python_helper_and_covers_everything():
    for total, granule, parts in [(4096, 8, 8), (520, 8, 3), (256, 1, 8), (16, 8, 4), (0, 8, 2), (40, 8, 8)]:
        covered = 0
        for r in range(parts):
            rc, b, n = _c_range(total, granule, parts, r)
            assert rc == _cabi.OK
            lo, hi = shard_range(total, r, parts, granule)
            assert (b, b + n) == (lo, hi) and n % granule == 0 and b == covered
            covered += n
        assert covered == total
    assert _c_range(100, 8, 4, 0)[0] == _cabi.ERR_UNSUPPORTED       # not a multiple of the granule
    assert _c_range(64, 8, 4, 4)[0] == _cabi.ERR_INVALID_ARG


def test_clone_is_an_independent_host_copy():
    m = sb.BlockwiseSpMatrix().init_random(128, 96, 32, 1, 0.25, True, 3, values="uniform")
    h = C.c_void_p()
    assert _cabi.lib().shflbw_matrix_clone(m._h, C.byref(h)) == _cabi.OK
    try:
        lib = _cabi.lib()
        assert lib.shflbw_matrix_nnzb(h) == m.nnzb and lib.shflbw_matrix_on_device(h) == 0
        n = m.nnzb
        assert np.array_equal(np.ctypeslib.as_array(lib.shflbw_matrix_indices(h), (n,)), m.indices)
        assert lib.shflbw_matrix_validate(h) == _cabi.OK
    finally:
        _cabi.lib().shflbw_matrix_destroy(h)


@pytest.mark.gpu
def test_sharded_spmm_and_spconv_equal_the_single_device_results():
    import torch

    import oracle_api as oa
    from conftest import assert_close_fp16
    from gpu_util import host
    lib = _cabi.lib()
    ndev = torch.cuda.device_count()
    devs = [0, 1] if ndev >= 2 else [0, 0]
    ids = (C.c_int * 2)(*devs)

    def on(dev_index, a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(f"cuda:{dev_index}").view(torch.float16)

    # ---- SpMM: 1000 dense columns -> shards of 504 and 496
    M, K, N, V = 256, 320, 1000, 64
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, 1, 0.3, True, 21, values="uniform")
    B = sb.uniform_half(22, K * N).reshape(K, N)
    mg = C.c_void_p()
    assert lib.shflbw_multi_create(m._h, ids, 2, C.byref(mg)) == _cabi.OK
    try:
        assert lib.shflbw_multi_shards(mg) == 2
        parts = [_c_range(N, 8, 2, r)[1:] for r in range(2)]
        assert [p[1] for p in parts] == [504, 496]
        Bs = [on(devs[g], B[:, b:b + n]) for g, (b, n) in enumerate(parts)]
        Ds = [torch.full((M, n), float("nan"), dtype=torch.float16, device=f"cuda:{devs[g]}") for g, (b, n) in enumerate(parts)]
        ns = (C.c_int * 2)(*[n for _, n in parts])
        bp = (C.c_void_p * 2)(*[t.data_ptr() for t in Bs])
        dp = (C.c_void_p * 2)(*[t.data_ptr() for t in Ds])
        assert lib.shflbw_multi_spmm_init(mg, ns, bp, dp, 1.0) == _cabi.OK
        before = torch.cuda.current_device()
        assert lib.shflbw_multi_exec(mg) == _cabi.OK
        ms = C.c_float()
        assert lib.shflbw_multi_sync(mg, C.byref(ms)) == _cabi.OK and ms.value > 0
        assert torch.cuda.current_device() == before            # the caller's device is restored
        got = np.concatenate([host(d) for d in Ds], axis=1)
        ref = oa.spmm_ref(M, N, V, m.indptr, m.indices, m.values, m.row_permute_ids, B)
        assert_close_fp16(got, ref, what="SpMM over two column shards")
    finally:
        lib.shflbw_multi_destroy(mg)

    # ---- SpConv: 12 images -> 6 + 6
    Bn, H, W, Cc, F = 12, 9, 7, 32, 128
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, 64, 1, 0.25, True, 23, values="uniform")
    x = sb.uniform_half(24, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    assert lib.shflbw_multi_create(f._h, ids, 2, C.byref(mg)) == _cabi.OK
    try:
        parts = [_c_range(Bn, 1, 2, r)[1:] for r in range(2)]
        xs = [on(devs[g], x[b:b + n]) for g, (b, n) in enumerate(parts)]
        os_ = [torch.full((n, H, W, F), float("nan"), dtype=torch.float16, device=f"cuda:{devs[g]}") for g, (b, n) in enumerate(parts)]
        ns = (C.c_int * 2)(*[n for _, n in parts])
        ip = (C.c_void_p * 2)(*[t.data_ptr() for t in xs])
        op = (C.c_void_p * 2)(*[t.data_ptr() for t in os_])
        assert lib.shflbw_multi_spconv_init(mg, ns, H, W, 1, ip, op, 0.5) == _cabi.OK
        assert lib.shflbw_multi_exec(mg) == _cabi.OK
        assert lib.shflbw_multi_sync(mg, None) == _cabi.OK
        got = np.concatenate([host(o) for o in os_], axis=0)
        ref = oa.spconv_ref_nhwc(Bn, H, W, Cc, F, 3, 3, 1, 64, f.indptr, f.indices, f.values, f.row_permute_ids, x, 0.5)
        assert_close_fp16(got, ref, what="SpConv over two batch shards")
    finally:
        lib.shflbw_multi_destroy(mg)
