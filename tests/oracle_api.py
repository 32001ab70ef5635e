"""ctypes access to the CPU oracle (oracle/liboracle.so) and, when built, to the unmodified
reference (oracle/_ref/*.so).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
ORACLE_LIB = ORACLE_DIR / "liboracle.so"
REF_HOST_LIB = ORACLE_DIR / "_ref" / "libshflbw_ref_host.so"
REF_GPU_LIB = ORACLE_DIR / "_ref" / "libshflbw_ref_gpu.so"

_P = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)


def build_oracle() -> None:
    src = ORACLE_DIR / "shflbw_oracle.cc"
    if not ORACLE_LIB.exists() or ORACLE_LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), "liboracle.so"], check=True, capture_output=True)


_orc = None


def orc() -> C.CDLL:
    global _orc
    if _orc is None:
        build_oracle()
        l = C.CDLL(str(ORACLE_LIB))
        l.orc_random_mask.argtypes = [C.c_int] * 4 + [C.c_float, C.c_uint] + [C.c_void_p] * 3
        l.orc_row_permutation.argtypes = [C.c_int, C.c_uint, C.c_void_p]
        l.orc_fill_int9.argtypes = [C.c_int64, C.c_void_p]
        l.orc_srand.argtypes = [C.c_uint]
        l.orc_achieved_density.restype = C.c_float
        l.orc_achieved_density.argtypes = [C.c_int] * 5
        l.orc_dump_text.restype = C.c_int64
        l.orc_dump_text.argtypes = [C.c_int] * 6 + [C.c_void_p] * 5 + [C.c_int64]
        l.orc_meta_image.restype = C.c_int64
        l.orc_meta_image.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        l.orc_spmm_ref.argtypes = [C.c_int] * 3 + [C.c_void_p] * 5 + [C.c_float, C.c_void_p, C.c_float, C.c_void_p, C.c_int]
        l.orc_spconv_ref_chwn.argtypes = [C.c_int] * 9 + [C.c_void_p] * 6 + [C.c_int]
        l.orc_spconv_ref_nhwc.argtypes = [C.c_int] * 9 + [C.c_void_p] * 5 + [C.c_float, C.c_void_p, C.c_int]
        l.orc_expand_block_columns.argtypes = [C.c_int] * 3 + [C.c_void_p] * 6
        l.orc_check_equal_ref_rule.restype = C.c_int64
        l.orc_check_equal_ref_rule.argtypes = [C.c_int64, C.c_void_p, C.c_void_p]
        _orc = l
    return _orc


# ---- oracle wrappers -----------------------------------------------------------------

def random_mask(nrow, ncol, brow, bcol, density, seed):
    X, Y = nrow // brow, ncol // bcol
    indptr = np.zeros(X + 1, np.int32)
    indices = np.zeros(X * Y, np.int32)
    nnzb = C.c_int()
    rc = orc().orc_random_mask(nrow, ncol, brow, bcol, density, seed, C.addressof(nnzb), _P(indptr), _P(indices))
    assert rc == 0, rc
    return nnzb.value, indptr, indices[: nnzb.value].copy()


def row_permutation(nrow, seed):
    perm = np.zeros(nrow, np.int32)
    orc().orc_row_permutation(nrow, seed, _P(perm))
    return perm


def fill_int9(n):
    out = np.zeros(n, np.uint16)
    orc().orc_fill_int9(n, _P(out))
    return out.view(np.float16)


def srand(seed=1):
    orc().orc_srand(seed)


def dump_text(nrow, ncol, brow, indptr, indices, values, perm, bcol=1):
    nnzb = int(indices.size)
    v = np.ascontiguousarray(values).view(np.uint16)
    args = (nrow, ncol, nnzb, brow, bcol, 0 if perm is None else 1, _P(indptr), _P(indices), _P(v), _P(perm))
    n = orc().orc_dump_text(*args, None, 0)
    buf = C.create_string_buffer(n)
    orc().orc_dump_text(*args, C.cast(buf, C.c_void_p), n)
    return buf.raw


def meta_image(indptr, indices, perm, bcol=1):
    n_perm = 0 if perm is None else int(perm.size)
    out = np.zeros(indptr.size + indices.size + n_perm + 32, np.int32)
    n = orc().orc_meta_image(int(indptr.size), _P(indptr), int(indices.size), _P(indices), bcol, n_perm, _P(perm), _P(out))
    return out[:n].copy()


def expand_block_columns(brow, bcol, indptr, indices, values):
    """brow x bcol blocks as brow x 1 blocks: (indptr, indices, values) for the other functions here."""
    indptr = np.ascontiguousarray(indptr, np.int32)
    indices = np.ascontiguousarray(indices, np.int32)
    v = np.ascontiguousarray(values).view(np.uint16)
    ip1, ix1, v1 = np.zeros_like(indptr), np.zeros(indices.size * bcol, np.int32), np.zeros_like(v)
    orc().orc_expand_block_columns(indptr.size - 1, brow, bcol, _P(indptr), _P(indices), _P(v), _P(ip1), _P(ix1), _P(v1))
    return ip1, ix1, v1.view(np.float16)


def spmm_ref(M, N, brow, indptr, indices, values, perm, B, alpha=1.0, Cm=None, beta=0.0, threads=8):
    D = np.zeros((M, N), np.float32)
    v = np.ascontiguousarray(values).view(np.uint16)
    b = np.ascontiguousarray(B).view(np.uint16)
    c = None if Cm is None else np.ascontiguousarray(Cm).view(np.uint16)
    orc().orc_spmm_ref(M, N, brow, _P(indptr), _P(indices), _P(v), _P(perm), _P(b), alpha, _P(c), beta, _P(D), threads)
    return D


def spconv_ref_chwn(Bn, H, W, Cc, F, R, S, stride, brow, indptr, indices, values, perm, ifmap, threads=8):
    out = np.zeros((F, H, W, Bn), np.float32)
    v = np.ascontiguousarray(values).view(np.uint16)
    x = np.ascontiguousarray(ifmap).view(np.uint16)
    orc().orc_spconv_ref_chwn(Bn, H, W, Cc, F, R, S, stride, brow, _P(indptr), _P(indices), _P(v), _P(perm), _P(x), _P(out), threads)
    return out


def spconv_ref_nhwc(Bn, Hin, Win, Cc, F, R, S, stride, brow, indptr, indices, values, perm, ifmap, alpha=1.0, threads=8):
    Ho, Wo = -(-Hin // stride), -(-Win // stride)
    out = np.zeros((Bn, Ho, Wo, F), np.float32)
    v = np.ascontiguousarray(values).view(np.uint16)
    x = np.ascontiguousarray(ifmap).view(np.uint16)
    orc().orc_spconv_ref_nhwc(Bn, Hin, Win, Cc, F, R, S, stride, brow, _P(indptr), _P(indices), _P(v), _P(perm), _P(x), alpha, _P(out), threads)
    return out


def ref_rule_violations(res_fp16, ref_f32):
    r = np.ascontiguousarray(res_fp16).view(np.uint16)
    f = np.ascontiguousarray(ref_f32, dtype=np.float32)
    return orc().orc_check_equal_ref_rule(r.size, _P(r), _P(f))


# ---- unmodified reference (present only when oracle/_ref was built) --------------------

_ref_host = None


def ref_host():
    """The reference's own host code, or None when oracle/_ref is absent."""
    global _ref_host
    if _ref_host is None:
        if not REF_HOST_LIB.exists():
            return None
        l = C.CDLL(str(REF_HOST_LIB))
        l.ref_matrix_init_random.restype = C.c_void_p
        l.ref_matrix_init_random.argtypes = [C.c_int] * 4 + [C.c_float, C.c_int, C.c_uint]
        l.ref_filter_init_random.restype = C.c_void_p
        l.ref_filter_init_random.argtypes = [C.c_int] * 6 + [C.c_float, C.c_int, C.c_uint]
        l.ref_matrix_free.argtypes = [C.c_void_p]
        l.ref_matrix_nnzb.argtypes = [C.c_void_p]
        l.ref_matrix_density.restype = C.c_float
        l.ref_matrix_density.argtypes = [C.c_void_p]
        l.ref_matrix_config_str.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        l.ref_matrix_arrays.argtypes = [C.c_void_p] * 5
        l.ref_matrix_dump.restype = C.c_int64
        l.ref_matrix_dump.argtypes = [C.c_void_p, C.c_char_p, C.c_int64]
        l.ref_matrix_load.restype = C.c_void_p
        l.ref_matrix_load.argtypes = [C.c_char_p, C.c_int64]
        l.ref_matrix_meta_image.restype = C.c_int64
        l.ref_matrix_meta_image.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        l.ref_spmm_host_reference.argtypes = [C.c_int] * 5 + [C.c_void_p] * 5 + [C.c_float, C.c_void_p, C.c_float, C.c_void_p]
        l.ref_spconv_host_reference.argtypes = [C.c_int] * 10 + [C.c_void_p] * 6
        l.ref_spmm_host_reference_blocks.argtypes = [C.c_int] * 6 + [C.c_void_p] * 5 + [C.c_float, C.c_void_p, C.c_float, C.c_void_p]
        l.ref_spconv_host_reference_blocks.argtypes = [C.c_int] * 11 + [C.c_void_p] * 6
        _ref_host = l
    return _ref_host


class RefMatrix:
    """A BlockwiseSpMatrix<half> / BlockwiseSpFilter<half> built by the reference itself."""

    def __init__(self, handle, nrow, brow, permute, bcol=1):
        self.h, self.nrow, self.brow, self.permute, self.bcol = handle, nrow, brow, permute, bcol
        l = ref_host()
        self.nnzb = l.ref_matrix_nnzb(handle)
        self.density = l.ref_matrix_density(handle)
        self.indptr = np.zeros(nrow // brow + 1, np.int32)
        self.indices = np.zeros(self.nnzb, np.int32)
        v = np.zeros(self.nnzb * brow * bcol, np.uint16)
        self.perm = np.zeros(nrow, np.int32) if permute else None
        l.ref_matrix_arrays(handle, _P(self.indptr), _P(self.indices), _P(v), _P(self.perm))
        self.values = v.view(np.float16)
        buf = C.create_string_buffer(256)
        l.ref_matrix_config_str(handle, buf, 256)
        self.config_str = buf.value.decode()

    @classmethod
    def init_random(cls, nrow, ncol, brow, density, permute, seed, bcol=1):
        return cls(ref_host().ref_matrix_init_random(nrow, ncol, brow, bcol, density, int(permute), seed), nrow, brow, permute, bcol)

    @classmethod
    def filter_init_random(cls, F, R, S, Cc, brow, density, permute, seed, bcol=1):
        return cls(ref_host().ref_filter_init_random(F, R, S, Cc, brow, bcol, density, int(permute), seed), F, brow, permute, bcol)

    def dump(self):
        l = ref_host()
        n = l.ref_matrix_dump(self.h, None, 0)
        buf = C.create_string_buffer(n)
        l.ref_matrix_dump(self.h, buf, n)
        return buf.raw

    def meta_image(self):  # needs a GPU
        l = ref_host()
        out = np.zeros(self.indptr.size + self.indices.size + self.nrow + 64, np.int32)
        n = l.ref_matrix_meta_image(self.h, _P(out), out.size)
        return out[:n].copy()

    def __del__(self):
        try:
            ref_host().ref_matrix_free(self.h)
        except Exception:
            pass


def ref_spmm_host_reference(M, K, N, brow, indptr, indices, values, perm, B, alpha=1.0, Cm=None, beta=0.0, bcol=1):
    D = np.zeros((M, N), np.float32)
    v = np.ascontiguousarray(values).view(np.uint16)
    b = np.ascontiguousarray(B).view(np.uint16)
    c = None if Cm is None else np.ascontiguousarray(Cm).view(np.uint16)
    ref_host().ref_spmm_host_reference_blocks(M, K, N, brow, bcol, int(indices.size), _P(indptr), _P(indices), _P(v),
                                              _P(perm), _P(b), alpha, _P(c), beta, _P(D))
    return D


def ref_spconv_host_reference(Bn, H, W, Cc, F, R, S, stride, brow, indptr, indices, values, perm, ifmap_chwn, bcol=1):
    out = np.zeros((F, H, W, Bn), np.float32)
    v = np.ascontiguousarray(values).view(np.uint16)
    x = np.ascontiguousarray(ifmap_chwn).view(np.uint16)
    ref_host().ref_spconv_host_reference_blocks(Bn, H, W, Cc, F, R, S, stride, brow, bcol, int(indices.size),
                                                _P(indptr), _P(indices), _P(v), _P(perm), _P(x), _P(out))
    return out


_ref_gpu = None


def ref_gpu():
    """The reference's CUDA kernels compiled for sm_100a, or None."""
    global _ref_gpu
    if _ref_gpu is None:
        if not REF_GPU_LIB.exists():
            return None
        l = C.CDLL(str(REF_GPU_LIB))
        l.ref_gpu_spmm_config_name.restype = C.c_char_p
        l.ref_gpu_conv_config_name.restype = C.c_char_p
        l.ref_gpu_spmm.argtypes = [C.c_int] * 6 + [C.c_void_p] * 6 + [C.c_int, C.c_int, C.POINTER(C.c_float)]
        l.ref_gpu_spconv.argtypes = [C.c_int] * 11 + [C.c_void_p] * 6 + [C.c_int, C.c_int, C.POINTER(C.c_float)]
        if hasattr(l, "ref_gpu_spmm_rotating"):
            l.ref_gpu_spmm_rotating.argtypes = [C.c_int] * 6 + [C.c_void_p] * 6 + [C.c_int] * 3 + [C.POINTER(C.c_float)]
            l.ref_gpu_spconv_rotating.argtypes = [C.c_int] * 11 + [C.c_void_p] * 6 + [C.c_int] * 3 + [C.POINTER(C.c_float)]
        _ref_gpu = l
    return _ref_gpu


def ref_gpu_spmm_configs(V):
    l = ref_gpu()
    return [(i, l.ref_gpu_spmm_config_name(i).decode()) for i in range(l.ref_gpu_num_spmm_configs())
            if l.ref_gpu_spmm_config_V(i) == V]


def ref_gpu_conv_configs(V):
    l = ref_gpu()
    return [(i, l.ref_gpu_conv_config_name(i).decode()) for i in range(l.ref_gpu_num_conv_configs())
            if l.ref_gpu_conv_config_V(i) == V]


def ref_gpu_spmm(cfg, M, K, N, brow, indptr, indices, values, perm, B_dev_ptr, D_dev_ptr, warmup=0, repeat=0):
    ms = C.c_float(0)
    v = np.ascontiguousarray(values).view(np.uint16)
    rc = ref_gpu().ref_gpu_spmm(cfg, M, K, N, brow, int(indices.size), _P(indptr), _P(indices), _P(v), _P(perm),
                                B_dev_ptr, D_dev_ptr, warmup, repeat, C.byref(ms))
    return rc, ms.value


def ref_gpu_spconv(cfg, Bn, H, W, Cc, F, R, S, stride, brow, indptr, indices, values, perm, in_ptr, out_ptr,
                   warmup=0, repeat=0):
    ms = C.c_float(0)
    v = np.ascontiguousarray(values).view(np.uint16)
    rc = ref_gpu().ref_gpu_spconv(cfg, Bn, H, W, Cc, F, R, S, stride, brow, int(indices.size), _P(indptr),
                                  _P(indices), _P(v), _P(perm), in_ptr, out_ptr, warmup, repeat, C.byref(ms))
    return rc, ms.value


def _ptr_array(ptrs):
    return (C.c_void_p * len(ptrs))(*ptrs)


def ref_gpu_spmm_rotating(cfg, M, K, N, brow, indptr, indices, values, perm, B_ptrs, D_ptrs, warmup, repeat):
    """Mean time (ms) of the reference SpMM kernel over `repeat` launches that rotate the buffer pairs."""
    ms = C.c_float(0)
    v = np.ascontiguousarray(values).view(np.uint16)
    rc = ref_gpu().ref_gpu_spmm_rotating(cfg, M, K, N, brow, int(indices.size), _P(indptr), _P(indices), _P(v), _P(perm),
                                         _ptr_array(B_ptrs), _ptr_array(D_ptrs), len(B_ptrs), warmup, repeat, C.byref(ms))
    return rc, ms.value


def ref_gpu_spconv_rotating(cfg, Bn, H, W, Cc, F, R, S, stride, brow, indptr, indices, values, perm, in_ptrs, out_ptrs,
                            warmup, repeat):
    ms = C.c_float(0)
    v = np.ascontiguousarray(values).view(np.uint16)
    rc = ref_gpu().ref_gpu_spconv_rotating(cfg, Bn, H, W, Cc, F, R, S, stride, brow, int(indices.size), _P(indptr),
                                           _P(indices), _P(v), _P(perm), _ptr_array(in_ptrs), _ptr_array(out_ptrs),
                                           len(in_ptrs), warmup, repeat, C.byref(ms))
    return rc, ms.value
