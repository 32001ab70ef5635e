"""Host-side mirror of the reference's operator interface on top of the C ABI.

Same names, argument meaning and lifetimes as the reference's C++ API so that tests read
like the reference's own (paths relative to the reference project):

  BlockwiseSpMatrix   block_sparse/spmm/blockwise_format.h:13-68
  BlockwiseSpFilter   block_sparse/spconv/blockwise_format.h:16-27
  SpmmBlockwiseOp / SpmmBlockwiseInitFn / SpmmBlockwiseExecFn
                      block_sparse/spmm/blockwise_op.h:19-52, 180-209
  SpconvBlockwiseOp / SpconvBlockwiseInitFn / SpconvBlockwiseExecFn
                      block_sparse/spconv/blockwise_op.h:19-50, 161-187

Differences, all deliberate: errors raise ShflbwError instead of exit()/assert; alpha is
honoured; SpConv activations are NHWC; device buffers are anything with `.data_ptr()`
(e.g. a torch CUDA tensor) or a raw integer device address.  All compute runs in the CUDA
library; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _cabi
from ._cabi import (KERNEL_AUTO, KERNEL_SIMT, KERNEL_TCGEN05, VALUES_INT9_LIBC, VALUES_UNIFORM,
                    ShflbwError, SpconvState, SpmmState, check)

_VALUE_MODES = {"int9": VALUES_INT9_LIBC, "uniform": VALUES_UNIFORM}


def _ptr(x) -> Optional[int]:
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    return int(x)


def _stream_ptr(stream) -> Optional[int]:
    if stream is None:
        return None
    if hasattr(stream, "cuda_stream"):
        return int(stream.cuda_stream)
    return int(stream)


def uniform_half(stream_seed: int, n: int, offset: int = 0) -> np.ndarray:
    """The library's seeded fp16 uniform[-1,1) stream (SHFLBW_VALUES_UNIFORM), in numpy.

    value i = rn_fp16(2*u - 1), u = (splitmix64(seed*2^32 + i) >> 40) / 2^24.  Used by tests and
    the benchmark to make dense operands; bit-identical to the C++ generator.
    """
    with np.errstate(over="ignore"):
        z = (np.uint64(stream_seed) << np.uint64(32)) + np.arange(offset, offset + n, dtype=np.uint64)
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = (z >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return (np.float32(2.0) * u - np.float32(1.0)).astype(np.float16)


class BlockwiseSpMatrix:
    """Shfl-BW sparse matrix: V x 1 vector-wise block CSR plus an optional row permutation."""

    def __init__(self):
        self._h = C.c_void_p()
        self.initialized = False

    # -- lifetime ---------------------------------------------------------------------
    def _reset(self):
        if self._h:
            _cabi.lib().shflbw_matrix_destroy(self._h)
        self._h = C.c_void_p()
        self.initialized = False

    def __del__(self):
        try:
            self._reset()
        except Exception:
            pass

    # -- builders ---------------------------------------------------------------------
    def init_random(self, nrow, ncol, brow, bcol, expected_density, row_permute, seed, values="int9"):
        self._reset()
        check(_cabi.lib().shflbw_matrix_create_random(nrow, ncol, brow, bcol, expected_density,
                                                      int(bool(row_permute)), seed, _VALUE_MODES[values],
                                                      C.byref(self._h)), "init_random")
        self.initialized = True
        return self

    @classmethod
    def from_arrays(cls, nrow, ncol, brow, indptr, indices, values, row_permute_ids=None, bcol=1):
        """Copy caller arrays.  With bcol > 1 the blocks are brow x bcol: `indices` counts in units
        of bcol columns and `values` holds each block column by column (blockwise_format.h:286-297)."""
        self = cls()
        indptr = np.ascontiguousarray(indptr, dtype=np.int32)
        indices = np.ascontiguousarray(indices, dtype=np.int32)
        values = np.ascontiguousarray(values).view(np.uint16).reshape(-1)
        perm = None if row_permute_ids is None else np.ascontiguousarray(row_permute_ids, dtype=np.int32)
        if indptr.size != (nrow // max(brow, 1)) + 1:
            raise ShflbwError(_cabi.ERR_BAD_FORMAT, "from_arrays", "indptr length")
        nnzb = int(indices.size)
        if values.size != nnzb * brow * bcol or (perm is not None and perm.size != nrow):
            raise ShflbwError(_cabi.ERR_BAD_FORMAT, "from_arrays", "array sizes")
        vp = values.ctypes.data if nnzb else None
        check(_cabi.lib().shflbw_matrix_create_from_block_arrays(
            nrow, ncol, brow, bcol, nnzb, indptr.ctypes.data, indices.ctypes.data if nnzb else None, vp,
            None if perm is None else perm.ctypes.data, C.byref(self._h)), "from_arrays")
        self.initialized = True
        return self

    def load(self, text):
        """Load from dumped text (str/bytes), as BlockwiseSpMatrix::load(std::istream&)."""
        data = text.encode() if isinstance(text, str) else bytes(text)
        self._reset()
        check(_cabi.lib().shflbw_matrix_load_text(data, len(data), C.byref(self._h)), "load")
        self.initialized = True
        return self

    def dump(self) -> bytes:
        need = C.c_size_t()
        l = _cabi.lib()
        check(l.shflbw_matrix_dump_text(self._h, None, 0, C.byref(need)), "dump")
        buf = C.create_string_buffer(need.value)
        check(l.shflbw_matrix_dump_text(self._h, buf, need.value, C.byref(need)), "dump")
        return buf.raw

    def validate(self):
        check(_cabi.lib().shflbw_matrix_validate(self._h), "validate")

    def transform_and_sync_device(self):
        check(_cabi.lib().shflbw_matrix_to_device(self._h), "transform_and_sync_device")

    def device_status(self):
        check(_cabi.lib().shflbw_matrix_device_status(self._h), "device_status")

    # -- fields -----------------------------------------------------------------------
    nrow = property(lambda s: _cabi.lib().shflbw_matrix_nrow(s._h))
    ncol = property(lambda s: _cabi.lib().shflbw_matrix_ncol(s._h))
    nnzb = property(lambda s: _cabi.lib().shflbw_matrix_nnzb(s._h))
    brow = property(lambda s: _cabi.lib().shflbw_matrix_brow(s._h))
    bcol = property(lambda s: _cabi.lib().shflbw_matrix_bcol(s._h))
    seed = property(lambda s: _cabi.lib().shflbw_matrix_seed(s._h))
    density = property(lambda s: _cabi.lib().shflbw_matrix_density(s._h))
    row_permute = property(lambda s: bool(_cabi.lib().shflbw_matrix_row_permute(s._h)))
    config_str = property(lambda s: _cabi.lib().shflbw_matrix_config_str(s._h).decode())
    device_synced = property(lambda s: bool(_cabi.lib().shflbw_matrix_on_device(s._h)))

    def _arr(self, fn, n, dtype):
        p = fn(self._h)
        if not p or n == 0:
            return np.zeros(0, dtype)
        return np.ctypeslib.as_array(p, shape=(n,)).astype(dtype, copy=True)

    @property
    def indptr(self):
        return self._arr(_cabi.lib().shflbw_matrix_indptr, self.nrow // self.brow + 1, np.int32)

    @property
    def indices(self):
        return self._arr(_cabi.lib().shflbw_matrix_indices, self.nnzb, np.int32)

    @property
    def values(self):
        return self._arr(_cabi.lib().shflbw_matrix_values, self.nnzb * self.brow * self.bcol, np.uint16).view(np.float16)

    @property
    def row_permute_ids(self):
        if not self.row_permute:
            return np.zeros(0, np.int32)
        return self._arr(_cabi.lib().shflbw_matrix_row_permute_ids, self.nrow, np.int32)

    @property
    def meta_h(self):
        n = C.c_size_t()
        p = _cabi.lib().shflbw_matrix_meta_image(self._h, C.byref(n))
        return np.ctypeslib.as_array(p, shape=(n.value,)).astype(np.int32, copy=True)


class BlockwiseSpFilter(BlockwiseSpMatrix):
    """Sparse conv filter F x R x S x C viewed as the matrix F x (R*S*C), k = (r*S+s)*C + c."""

    def init_random(self, F, R, S, C_, brow, bcol, expected_density, filter_permute, seed, values="int9"):
        self._reset()
        check(_cabi.lib().shflbw_filter_create_random(F, R, S, C_, brow, bcol, expected_density,
                                                      int(bool(filter_permute)), seed, _VALUE_MODES[values],
                                                      C.byref(self._h)), "init_random")
        self.initialized = True
        return self

    @classmethod
    def from_arrays(cls, F, R, S, C_, brow, indptr, indices, values, row_permute_ids=None, bcol=1):
        self = super().from_arrays(F, R * S * C_, brow, indptr, indices, values, row_permute_ids, bcol)
        check(_cabi.lib().shflbw_matrix_set_filter_shape(self._h, F, R, S, C_), "set_filter_shape")
        return self

    def _shape(self):
        v = [C.c_int() for _ in range(4)]
        check(_cabi.lib().shflbw_matrix_filter_shape(self._h, *[C.byref(x) for x in v]), "filter_shape")
        return tuple(x.value for x in v)

    def fold_input_order(self, producer: "BlockwiseSpMatrix") -> "BlockwiseSpFilter":
        """This filter with its input channels renumbered to `producer`'s stored filter order
        (for chained layers: the producer's output is consumed without its inverse permutation)."""
        out = BlockwiseSpFilter()
        check(_cabi.lib().shflbw_filter_fold_input_order(self._h, producer._h, C.byref(out._h)), "fold_input_order")
        out.initialized = True
        return out

    F = property(lambda s: s._shape()[0])
    R = property(lambda s: s._shape()[1])
    S = property(lambda s: s._shape()[2])
    C = property(lambda s: s._shape()[3])


# ------------------------------------------------------------------------------- SpMM --

class SpmmBlockwiseOp:
    """D = alpha * A_sparse . B + beta * C  (fp16 in, fp32 accumulate, fp16 out)."""

    def __init__(self, kernel: int = KERNEL_AUTO):
        self._state = SpmmState()
        self._kernel = kernel
        self._keep = None

    def initialize(self, spmat: BlockwiseSpMatrix, N: int, B, *rest):
        """initialize(spmat, N, B, D) | (spmat, N, B, C, D) [alpha=beta=1] |
        (spmat, N, B, alpha, C, beta, D) -- the three overloads of the reference."""
        if len(rest) == 1:
            alpha, Cm, beta, D = 1.0, None, 0.0, rest[0]
        elif len(rest) == 2:
            alpha, Cm, beta, D = 1.0, rest[0], 1.0, rest[1]
        elif len(rest) == 4:
            alpha, Cm, beta, D = rest
        else:
            raise TypeError("initialize(spmat, N, B, [alpha,] [C,] [beta,] D)")
        check(_cabi.lib().shflbw_spmm_init(spmat._h, N, _ptr(B), float(alpha), _ptr(Cm), float(beta), _ptr(D),
                                           self._kernel, C.byref(self._state)), "SpmmBlockwiseOp.initialize")
        self._keep = (spmat, B, Cm, D)  # state holds non-owning pointers
        return self

    def __call__(self, stream=None):
        check(_cabi.lib().shflbw_spmm_exec(C.byref(self._state), _stream_ptr(stream)), "SpmmBlockwiseOp()")

    @property
    def launches_per_exec(self) -> int:
        return _cabi.lib().shflbw_spmm_launches_per_exec(C.byref(self._state))


def SpmmBlockwiseInitFn(spmat, N, B, D, kernel: int = KERNEL_AUTO) -> SpmmBlockwiseOp:
    return SpmmBlockwiseOp(kernel).initialize(spmat, N, B, D)


def SpmmBlockwiseExecFn(state: SpmmBlockwiseOp, stream=None) -> None:
    state(stream)


def spmm_host(spmat: BlockwiseSpMatrix, N: int, B_host: np.ndarray, D_host: np.ndarray, alpha=1.0,
              C_host: Optional[np.ndarray] = None, beta=0.0) -> None:
    """End-to-end call with HOST buffers (numpy arrays or pinned torch CPU tensors)."""
    def hp(a):
        return None if a is None else (a.ctypes.data if isinstance(a, np.ndarray) else _ptr(a))
    check(_cabi.lib().shflbw_spmm_host(spmat._h, N, hp(B_host), float(alpha), hp(C_host), float(beta),
                                       hp(D_host)), "spmm_host")


# ----------------------------------------------------------------------------- SpConv --

class SpconvBlockwiseOp:
    """NHWC sparse convolution forward, pad R/2,S/2, Ho = ceil(Hin/stride)."""

    def __init__(self, kernel: int = KERNEL_AUTO):
        self._state = SpconvState()
        self._kernel = kernel
        self._keep = None

    def initialize(self, spfilter: BlockwiseSpFilter, B: int, H: int, W: int, stride: int, IFMap, OFMap,
                   alpha: float = 1.0):
        check(_cabi.lib().shflbw_spconv_init(spfilter._h, B, H, W, stride, _ptr(IFMap), _ptr(OFMap),
                                             float(alpha), self._kernel, C.byref(self._state)),
              "SpconvBlockwiseOp.initialize")
        self._keep = (spfilter, IFMap, OFMap)
        return self

    def __call__(self, stream=None):
        check(_cabi.lib().shflbw_spconv_exec(C.byref(self._state), _stream_ptr(stream)), "SpconvBlockwiseOp()")

    @property
    def launches_per_exec(self) -> int:
        return _cabi.lib().shflbw_spconv_launches_per_exec(C.byref(self._state))

    @property
    def out_hw(self):
        return self._state.Ho, self._state.Wo


# Chained conv layers: activations stay in the channel-major, halo-padded "chain buffer"
# layout between layers (see include/shflbw.h).  No counterpart in the reference.

def chain_buffer_elems(C_, H, W, B, R_consumer=1, S_consumer=1) -> int:
    return int(_cabi.lib().shflbw_chain_buffer_elems(C_, H, W, B, R_consumer, S_consumer))


def chain_import_nhwc(x_nhwc, B, H, W, C_, R_consumer, S_consumer, chain_buf, stream=None) -> None:
    check(_cabi.lib().shflbw_chain_import_nhwc(_ptr(x_nhwc), B, H, W, C_, R_consumer, S_consumer, _ptr(chain_buf),
                                               _stream_ptr(stream)), "chain_import_nhwc")


def chain_export_nhwc(chain_buf, B, H, W, F, R_halo, S_halo, producer, y_nhwc, stream=None) -> None:
    check(_cabi.lib().shflbw_chain_export_nhwc(_ptr(chain_buf), B, H, W, F, R_halo, S_halo,
                                               producer._h if producer is not None else None, _ptr(y_nhwc),
                                               _stream_ptr(stream)), "chain_export_nhwc")


class SpconvChainOp:
    """One chained layer: chain buffer in (halo of this filter), chain buffer out (halo of the
    consumer's R_next x S_next filter), optional fused ReLU; one kernel launch."""

    def __init__(self):
        self._state = SpconvState()
        self._keep = None

    def initialize(self, spfilter: BlockwiseSpFilter, B, H, W, stride, in_chain, out_chain, R_next=1, S_next=1,
                   alpha: float = 1.0, relu: bool = False):
        check(_cabi.lib().shflbw_spconv_chain_init(spfilter._h, B, H, W, stride, _ptr(in_chain), _ptr(out_chain),
                                                   R_next, S_next, float(alpha), int(bool(relu)),
                                                   C.byref(self._state)), "SpconvChainOp.initialize")
        self._keep = (spfilter, in_chain, out_chain)
        return self

    def set_residual(self, res_chain, residual_producer="same"):
        """out = relu?(alpha * conv + residual).  `res_chain` has the output's geometry; its channel
        order is that of `residual_producer`'s stored filters (None: logical order; "same": plane f
        is added to stored filter f)."""
        spfilter = self._keep[0]
        mp = None
        if residual_producer != "same":
            mp = np.empty(spfilter.nrow, np.int32)
            check(_cabi.lib().shflbw_chain_residual_map(spfilter._h, None if residual_producer is None
                                                        else residual_producer._h, mp.ctypes.data), "chain_residual_map")
        check(_cabi.lib().shflbw_spconv_chain_set_residual(spfilter._h, C.byref(self._state), _ptr(res_chain),
                                                           None if mp is None else mp.ctypes.data), "set_residual")
        self._keep = self._keep + (res_chain,)
        return self

    def __call__(self, stream=None):
        check(_cabi.lib().shflbw_spconv_exec(C.byref(self._state), _stream_ptr(stream)), "SpconvChainOp()")

    @property
    def launches_per_exec(self) -> int:
        return _cabi.lib().shflbw_spconv_launches_per_exec(C.byref(self._state))

    @property
    def out_hw(self):
        return self._state.Ho, self._state.Wo


def SpconvBlockwiseInitFn(spfilter, B, H, W, stride, IFMap, OFMap, kernel: int = KERNEL_AUTO):
    return SpconvBlockwiseOp(kernel).initialize(spfilter, B, H, W, stride, IFMap, OFMap)


def SpconvBlockwiseExecFn(state: SpconvBlockwiseOp, stream=None) -> None:
    state(stream)


def spconv_host(spfilter: BlockwiseSpFilter, B, H, W, stride, ifmap_host, ofmap_host, alpha=1.0) -> None:
    def hp(a):
        return a.ctypes.data if isinstance(a, np.ndarray) else _ptr(a)
    check(_cabi.lib().shflbw_spconv_host(spfilter._h, B, H, W, stride, hp(ifmap_host), hp(ofmap_host),
                                         float(alpha)), "spconv_host")
