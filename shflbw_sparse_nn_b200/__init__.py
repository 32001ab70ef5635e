"""B200-native (sm_100a) Shfl-BW block-sparse inference: format builder, SpMM, SpConv.

The compute path is the CUDA library `libshflbw_b200.so` (built in-tree by
`shflbw_sparse_nn_b200.build`); this package is the thin host-side mirror of the reference's
operator interface over that library's C ABI (include/shflbw.h).
"""
from ._cabi import (KERNEL_AUTO, KERNEL_SIMT, KERNEL_TCGEN05, VALUES_INT9_LIBC, VALUES_UNIFORM,
                    ShflbwError)
from .blockwise import (BlockwiseSpFilter, BlockwiseSpMatrix, SpconvBlockwiseExecFn, SpconvChainOp,
                        chain_buffer_elems, chain_export_nhwc, chain_import_nhwc,
                        SpconvBlockwiseInitFn, SpconvBlockwiseOp, SpmmBlockwiseExecFn,
                        SpmmBlockwiseInitFn, SpmmBlockwiseOp, spconv_host, spmm_host, uniform_half)

from .pruner import prune_conv_filter, prune_matrix

__all__ = [
    "prune_matrix", "prune_conv_filter",
    "BlockwiseSpMatrix", "BlockwiseSpFilter", "SpmmBlockwiseOp", "SpmmBlockwiseInitFn",
    "SpmmBlockwiseExecFn", "SpconvBlockwiseOp", "SpconvBlockwiseInitFn", "SpconvBlockwiseExecFn",
    "spmm_host", "spconv_host", "uniform_half", "ShflbwError",
    "SpconvChainOp", "chain_buffer_elems", "chain_import_nhwc", "chain_export_nhwc",
    "KERNEL_AUTO", "KERNEL_TCGEN05", "KERNEL_SIMT", "VALUES_INT9_LIBC", "VALUES_UNIFORM",
]
