"""ctypes binding of the C ABI declared in include/shflbw.h.

Loading fails loudly when the native library is missing: there is no Python or CPU
substitute for the CUDA path.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from .build import LIB_PATH

OK = 0
ERR_INVALID_ARG, ERR_BAD_FORMAT, ERR_UNSUPPORTED, ERR_CUDA = 1, 2, 3, 4
ERR_NOT_ON_DEVICE, ERR_DEVICE_TIMEOUT, ERR_IO, ERR_TOO_LARGE = 5, 6, 7, 8
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024
VALUES_INT9_LIBC, VALUES_UNIFORM = 0, 1
KERNEL_AUTO, KERNEL_TCGEN05, KERNEL_SIMT = 0, 1, 2


class ShflbwError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        super().__init__(f"{where}: status {status} ({detail})")


class SpmmState(C.Structure):
    """Mirror of shflbw_spmm_state_t."""
    _fields_ = [
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("V", C.c_int),
        ("num_row_blocks", C.c_int), ("kernel", C.c_int), ("tokens_per_cta", C.c_int),
        ("stages", C.c_int), ("producer_warps", C.c_int), ("variant", C.c_int), ("num_items", C.c_int),
        ("tiles_n", C.c_int),
        ("grid_x", C.c_uint), ("grid_y", C.c_uint), ("block_x", C.c_uint),
        ("shared_mem_size", C.c_size_t), ("init_success", C.c_int),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("B", C.c_void_p), ("C", C.c_void_p), ("D", C.c_void_p),
        ("blk_ptr", C.c_void_p), ("blk_idx", C.c_void_p), ("blk_val", C.c_void_p),
        ("perm", C.c_void_p), ("status_word", C.c_void_p),
        ("gather", C.c_int), ("tmap_b", C.c_ulonglong * 16),
    ]


class SpconvState(C.Structure):
    """Mirror of shflbw_spconv_state_t."""
    _fields_ = [
        ("B", C.c_int), ("Hin", C.c_int), ("Win", C.c_int), ("C", C.c_int), ("F", C.c_int),
        ("R", C.c_int), ("S", C.c_int), ("stride", C.c_int), ("Ho", C.c_int), ("Wo", C.c_int),
        ("V", C.c_int), ("Bp", C.c_int), ("kernel", C.c_int), ("tokens_per_cta", C.c_int),
        ("stages", C.c_int), ("producer_warps", C.c_int), ("variant", C.c_int), ("num_items", C.c_int),
        ("tiles_n", C.c_int),
        ("grid_x", C.c_uint), ("grid_y", C.c_uint), ("block_x", C.c_uint),
        ("shared_mem_size", C.c_size_t), ("init_success", C.c_int), ("alpha", C.c_float),
        ("ifmap", C.c_void_p), ("ofmap", C.c_void_p), ("staged_in", C.c_void_p),
        ("staged_out", C.c_void_p), ("staged_in_bytes", C.c_size_t), ("staged_out_bytes", C.c_size_t),
        ("blk_ptr", C.c_void_p), ("blk_idx", C.c_void_p), ("blk_val", C.c_void_p),
        ("perm", C.c_void_p), ("status_word", C.c_void_p),
        ("chain", C.c_int), ("out_R", C.c_int), ("out_S", C.c_int), ("relu", C.c_int),
        ("residual", C.c_void_p), ("residual_map", C.c_void_p),
    ]


_H = C.c_void_p  # opaque shflbw_matrix_t*
_PROTOS = {
    # name: (restype, argtypes)
    "shflbw_strerror": (C.c_char_p, [C.c_int]),
    "shflbw_last_cuda_error": (C.c_char_p, []),
    "shflbw_abi_version": (C.c_int, []),
    "shflbw_set_wait_limit_cycles": (C.c_int, [C.c_longlong]),
    "shflbw_matrix_create_random": (C.c_int, [C.c_int] * 4 + [C.c_float, C.c_int, C.c_uint, C.c_int, C.POINTER(_H)]),
    "shflbw_filter_create_random": (C.c_int, [C.c_int] * 6 + [C.c_float, C.c_int, C.c_uint, C.c_int, C.POINTER(_H)]),
    "shflbw_matrix_create_from_arrays": (C.c_int, [C.c_int] * 4 + [C.c_void_p] * 4 + [C.POINTER(_H)]),
    "shflbw_matrix_create_from_block_arrays": (C.c_int, [C.c_int] * 5 + [C.c_void_p] * 4 + [C.POINTER(_H)]),
    "shflbw_matrix_set_filter_shape": (C.c_int, [_H] + [C.c_int] * 4),
    "shflbw_matrix_load_text": (C.c_int, [C.c_char_p, C.c_size_t, C.POINTER(_H)]),
    "shflbw_matrix_load_file": (C.c_int, [C.c_char_p, C.POINTER(_H)]),
    "shflbw_matrix_dump_text": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "shflbw_matrix_dump_file": (C.c_int, [_H, C.c_char_p]),
    "shflbw_matrix_validate": (C.c_int, [_H]),
    "shflbw_matrix_destroy": (None, [_H]),
    "shflbw_matrix_nrow": (C.c_int, [_H]),
    "shflbw_matrix_ncol": (C.c_int, [_H]),
    "shflbw_matrix_nnzb": (C.c_int, [_H]),
    "shflbw_matrix_brow": (C.c_int, [_H]),
    "shflbw_matrix_bcol": (C.c_int, [_H]),
    "shflbw_matrix_row_permute": (C.c_int, [_H]),
    "shflbw_matrix_seed": (C.c_uint, [_H]),
    "shflbw_matrix_density": (C.c_float, [_H]),
    "shflbw_matrix_config_str": (C.c_char_p, [_H]),
    "shflbw_matrix_filter_shape": (C.c_int, [_H] + [C.POINTER(C.c_int)] * 4),
    "shflbw_matrix_indptr": (C.POINTER(C.c_int), [_H]),
    "shflbw_matrix_indices": (C.POINTER(C.c_int), [_H]),
    "shflbw_matrix_values": (C.POINTER(C.c_uint16), [_H]),
    "shflbw_matrix_row_permute_ids": (C.POINTER(C.c_int), [_H]),
    "shflbw_matrix_to_device": (C.c_int, [_H]),
    "shflbw_matrix_on_device": (C.c_int, [_H]),
    "shflbw_matrix_meta_image": (C.POINTER(C.c_int), [_H, C.POINTER(C.c_size_t)]),
    "shflbw_matrix_device_status": (C.c_int, [_H]),
    "shflbw_spmm_init": (C.c_int, [_H, C.c_int, C.c_void_p, C.c_float, C.c_void_p, C.c_float, C.c_void_p,
                                   C.c_int, C.POINTER(SpmmState)]),
    "shflbw_spmm_exec": (C.c_int, [C.POINTER(SpmmState), C.c_void_p]),
    "shflbw_spmm_host": (C.c_int, [_H, C.c_int, C.c_void_p, C.c_float, C.c_void_p, C.c_float, C.c_void_p]),
    "shflbw_spmm_host_copies_only": (C.c_int, [_H, C.c_int, C.c_void_p, C.c_void_p, C.c_int]),
    "shflbw_spmm_launches_per_exec": (C.c_int, [C.POINTER(SpmmState)]),
    "shflbw_spconv_init": (C.c_int, [_H, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                     C.c_float, C.c_int, C.POINTER(SpconvState)]),
    "shflbw_spconv_exec": (C.c_int, [C.POINTER(SpconvState), C.c_void_p]),
    "shflbw_spconv_host": (C.c_int, [_H, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float]),
    "shflbw_spconv_launches_per_exec": (C.c_int, [C.POINTER(SpconvState)]),
    "shflbw_chain_buffer_elems": (C.c_size_t, [C.c_int] * 6),
    "shflbw_chain_import_nhwc": (C.c_int, [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p, C.c_void_p]),
    "shflbw_chain_export_nhwc": (C.c_int, [C.c_void_p] + [C.c_int] * 6 + [_H, C.c_void_p, C.c_void_p]),
    "shflbw_filter_fold_input_order": (C.c_int, [_H, _H, C.POINTER(_H)]),
    "shflbw_spconv_chain_init": (C.c_int, [_H, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                           C.c_int, C.c_int, C.c_float, C.c_int, C.POINTER(SpconvState)]),
    "shflbw_chain_residual_map": (C.c_int, [_H, _H, C.c_void_p]),
    "shflbw_spconv_chain_set_residual": (C.c_int, [_H, C.POINTER(SpconvState), C.c_void_p, C.c_void_p]),
    "shflbw_shard_range": (C.c_int, [C.c_longlong, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]),
    "shflbw_matrix_clone": (C.c_int, [_H, C.POINTER(_H)]),
    "shflbw_multi_create": (C.c_int, [_H, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_void_p)]),
    "shflbw_multi_destroy": (None, [C.c_void_p]),
    "shflbw_multi_shards": (C.c_int, [C.c_void_p]),
    "shflbw_multi_spmm_init": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_float]),
    "shflbw_multi_spconv_init": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int,
                                           C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_float]),
    "shflbw_multi_exec": (C.c_int, [C.c_void_p]),
    "shflbw_multi_sync": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "shflbw_spconv_exec_static_scratch": (C.c_int, [_H, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                                    C.c_float, C.c_void_p]),
}

_lib = None


def exported_symbols() -> list[str]:
    """Every entry point include/shflbw.h declares (used by the symbol-export test)."""
    return sorted(_PROTOS)


def load_library(path) -> C.CDLL:
    """Load a build of the native library from `path` and set the prototypes of every declared
    entry point on it (AttributeError if one is not exported)."""
    path = Path(path)
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m shflbw_sparse_nn_b200.build` "
            "(there is no CPU fallback for the CUDA path)")
    handle = C.CDLL(str(path))
    for name, (res, args) in _PROTOS.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    return handle


def lib() -> C.CDLL:
    """Load (once) and return the native library; raises if it has not been built."""
    global _lib
    if _lib is None:
        _lib = load_library(LIB_PATH)
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        l = lib()
        detail = l.shflbw_strerror(status).decode()
        if status in (ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_TOO_LARGE):
            detail += "; " + l.shflbw_last_cuda_error().decode()
        raise ShflbwError(status, where, detail)
