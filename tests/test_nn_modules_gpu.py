"""The torch.nn front end (shflbw_sparse_nn_b200/nn.py) and the pruner, through the CUDA path:
a pruned operand must behave exactly like the masked dense layer.  References are fp32 torch
ops on the CPU over the same fp16-rounded weights and inputs; tolerance is the suite's
max(1e-2*|ref|, 1e-3)."""
import numpy as np
import pytest
import torch

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from gpu_util import run_spmm
from shflbw_sparse_nn_b200.nn import ShflBWConv2d, ShflBWLinear, densify
from shflbw_sparse_nn_b200.pruner import prune_matrix

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("V", [16, 32, 64, 128])
def test_pruned_matrix_through_the_cuda_kernel_equals_masked_dense_matmul(V):
    rng = np.random.default_rng(V)
    W = rng.normal(size=(2 * 128, 384)).astype(np.float32)
    m, info = prune_matrix(W, V=V, density=0.25, permute=True, seed=1)
    B = rng.uniform(-1, 1, (384, 200)).astype(np.float16)
    D, op = run_spmm(m, 200, B)
    assert op._state.kernel == sb.KERNEL_TCGEN05
    want = densify(m).astype(np.float32) @ B.astype(np.float32)
    assert_close_fp16(D, want, what=f"pruned V={V} vs masked dense")
    assert_close_fp16(D, oa.spmm_ref(m.nrow, 200, V, m.indptr, m.indices, m.values, m.row_permute_ids, B), what="vs oracle")


@pytest.mark.parametrize("bias", [False, True])
def test_linear_module_matches_the_masked_dense_layer(bias):
    torch.manual_seed(3)
    dense = torch.nn.Linear(320, 256, bias=bias)
    lin = ShflBWLinear.from_dense(dense, V=64, density=0.2)
    assert 0.2 < lin.info["retained"] <= 1.0
    x = (torch.rand(3, 37, 320) * 2 - 1).half()                     # 111 tokens: not a multiple of 8
    y = lin(x.cuda())
    torch.cuda.synchronize()
    lin.spmat.device_status()
    assert y.shape == (3, 37, 256) and y.dtype == torch.float16
    b = None if not bias else dense.bias.detach().half().float()
    want = torch.nn.functional.linear(x.float(), lin.dense_weight().float(), b)
    assert_close_fp16(y.cpu().numpy(), want.numpy(), abs_=2e-3, what="ShflBWLinear")
    # zero-copy entry: [in][tokens] -> [out][tokens]
    xt = x.reshape(-1, 320)[:104].t().contiguous().cuda()
    yt = lin.forward_feature_major(xt)
    torch.cuda.synchronize()
    assert_close_fp16(yt.cpu().numpy(), want.reshape(-1, 256)[:104].t().numpy(), abs_=2e-3, what="feature-major")


@pytest.mark.parametrize("k,stride", [(3, 1), (3, 2), (1, 1)])
def test_conv_module_matches_the_masked_dense_layer(k, stride):
    torch.manual_seed(5)
    dense = torch.nn.Conv2d(32, 128, k, stride=stride, padding=k // 2, bias=True)
    conv = ShflBWConv2d.from_dense(dense, V=64, density=0.3)
    x = (torch.rand(6, 32, 11, 9) * 2 - 1).half()
    y = conv(x.cuda().contiguous(memory_format=torch.channels_last))
    torch.cuda.synchronize()
    conv.spfilter.device_status()
    want = torch.nn.functional.conv2d(x.float(), conv.dense_weight().float(), dense.bias.detach().half().float(),
                                      stride=stride, padding=k // 2)
    assert y.shape == want.shape
    assert_close_fp16(y.cpu().numpy(), want.numpy(), abs_=2e-3, what=f"ShflBWConv2d k={k} stride={stride}")


def test_modules_refuse_what_the_kernels_cannot_run():
    with pytest.raises(ValueError):
        ShflBWConv2d.from_dense(torch.nn.Conv2d(32, 64, 3, padding=0), V=64, density=0.5)
    with pytest.raises(ValueError):
        ShflBWConv2d.from_dense(torch.nn.Conv2d(12, 64, 3, padding=1), V=64, density=0.5)
    lin = ShflBWLinear.from_dense(torch.nn.Linear(64, 64), V=64, density=0.5)
    with pytest.raises(TypeError):
        lin(torch.zeros(8, 64))
