"""The executed ResNet-50-shaped stack (shflbw_sparse_nn_b200.resnet50): 52 chained sparse
convolutions with folded channel orders, stride-2 layers, projection and identity shortcuts,
fused scale / residual add / ReLU, at a reduced spatial size so the CPU oracle finishes fast.

Every layer is checked on its own: its inputs are what the GPU produced for the layers before
it (exported to NHWC in logical channel order), its expected output is the CPU oracle's
convolution with the UNFOLDED filter, scaled, plus the shortcut, through ReLU.  A wrong channel
renumbering, residual map, halo or stride shows up at the first layer that uses it.  The final
NHWC output is compared as well, and a CUDA-graph replay must reproduce it bit for bit.
"""
import numpy as np
import pytest
import torch

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import dev, host
from shflbw_sparse_nn_b200.resnet50 import SparseResNet50

pytestmark = pytest.mark.gpu


def test_stack_layer_by_layer_against_the_oracle_and_graph_replay():
    Bn, hw = 8, 8
    net = SparseResNet50(Bn, hw=hw, density=0.2, V=64, seed=77)
    x = sb.uniform_half(9, Bn * hw * hw * 64).reshape(Bn, hw, hw, 64)
    net.x.copy_(dev(x))
    net.forward(torch.cuda.current_stream())
    torch.cuda.synchronize()
    net.check_status()
    outs = [host(net.layer_output_nhwc(i)) for i in range(len(net.specs))]
    torch.cuda.synchronize()
    for i, sp in enumerate(net.specs):
        f = net.filters[i]                                   # logical (unfolded) filter
        xin = x if sp.src < 0 else outs[sp.src]
        ref = oa.spconv_ref_nhwc(Bn, sp.Hin, sp.Hin, sp.C, sp.F, sp.R, sp.R, sp.stride, 64, f.indptr, f.indices,
                                 f.values, f.row_permute_ids, xin, alpha=net.alphas[i])
        if sp.residual is not None:
            ref = ref + (x if sp.residual < 0 else outs[sp.residual]).astype(np.float32)
        if sp.relu:
            ref = np.maximum(ref, 0.0)
        assert outs[i].shape == ref.shape
        # the fused epilogue rounds three times in fp16 (conv, scale, add): rel 1e-2 / abs 2e-3
        assert_close_fp16(outs[i], ref, abs_=2e-3, what=f"layer {i} {sp.name}")
    y1 = host(net.y)
    assert np.array_equal(y1.view(np.uint16), outs[-1].view(np.uint16))
    assert np.isfinite(y1.astype(np.float32)).all() and float(np.abs(y1.astype(np.float32)).max()) > 0.0
    replay = net.capture()
    net.y.zero_()
    replay()
    torch.cuda.synchronize()
    net.check_status()
    assert np.array_equal(host(net.y).view(np.uint16), y1.view(np.uint16))
    assert net.launches_per_forward == 54
