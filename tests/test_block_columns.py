"""brow x bcol blocks with bcol > 1 (block_sparse/spmm/blockwise_format.h stores them; the
reference's kernels assert bcol == 1, spmm/blockwise_op.h:86, so only its host code is a check).

CPU part: the builder, dump/load and the device images against the oracle, the oracle's
block-column expansion against the outputs of the reference's two host references committed
in tests/golden/block_column_cases.npz, and the 2 x 2 example of
example/spmatrix_dump_load.md.  GPU part: SpMM and SpConv on such matrices through the C ABI.
Bit-exact bar for the integer/index work; fp16 tolerance of conftest.assert_close_fp16 for
the kernels."""
import numpy as np
import pytest

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from conftest import assert_close_fp16
from shflbw_sparse_nn_b200.nn import densify

DOC_TEXT = "4\n4\n2\n2\n2\n0\n0 1 2 \n0 1 \n1 2 1 2 3 1 1 2 \n"   # example/spmatrix_dump_load.md:30-40
DOC_MATRIX = np.array([[1, 1, 0, 0], [2, 2, 0, 0], [0, 0, 3, 1], [0, 0, 1, 2]], np.float16)


def test_documented_2x2_example_loads_dumps_and_densifies():
    m = sb.BlockwiseSpMatrix().load(DOC_TEXT)
    assert (m.nrow, m.ncol, m.nnzb, m.brow, m.bcol, bool(m.row_permute)) == (4, 4, 2, 2, 2, False)
    assert m.dump().decode().split() == DOC_TEXT.split()
    assert m.dump() == oa.dump_text(4, 4, 2, m.indptr, m.indices, m.values, None, bcol=2)
    assert np.array_equal(densify(m), DOC_MATRIX)
    # the oracle reads the same matrix out of the same arrays
    ip, ix, v = oa.expand_block_columns(2, 2, m.indptr, m.indices, m.values)
    assert np.array_equal(oa.spmm_ref(4, 4, 2, ip, ix, v, None, np.eye(4, dtype=np.float16)), DOC_MATRIX.astype(np.float32))
    # with the documented permutation 0 3 1 2 the saved matrix has rows 0, 3 in the first block
    p = sb.BlockwiseSpMatrix.from_arrays(4, 4, 2, m.indptr, m.indices, m.values, np.array([0, 3, 1, 2], np.int32), bcol=2)
    assert np.array_equal(densify(p), DOC_MATRIX[[0, 2, 3, 1]])
    assert p.dump().decode().split()[-4:] == ["0", "3", "1", "2"]


@pytest.mark.parametrize("nrow,ncol,brow,bcol,d,perm,seed", [(256, 256, 32, 2, 0.1, True, 2021), (512, 320, 64, 4, 0.23, False, 5),
                                                             (64, 1024, 16, 8, 0.2, True, 2)])
def test_builder_matches_oracle(nrow, ncol, brow, bcol, d, perm, seed):
    n, indptr, indices = oa.random_mask(nrow, ncol, brow, bcol, d, seed)
    oa.srand(99)
    vals = oa.fill_int9(n * brow * bcol)
    oa.srand(99)
    m = sb.BlockwiseSpMatrix().init_random(nrow, ncol, brow, bcol, d, perm, seed, values="int9")
    assert m.nnzb == n and m.bcol == bcol
    assert np.array_equal(m.indptr, indptr) and np.array_equal(m.indices, indices)
    assert np.array_equal(m.values.view(np.uint16), vals.view(np.uint16))
    p = oa.row_permutation(nrow, seed) if perm else None
    assert m.dump() == oa.dump_text(nrow, ncol, brow, indptr, indices, vals, p, bcol=bcol)
    assert np.array_equal(m.meta_h, oa.meta_image(indptr, indices, p, bcol=bcol))   # indices * bcol
    again = sb.BlockwiseSpMatrix().load(m.dump())
    assert again.bcol == bcol and again.dump() == m.dump()
    m.validate()


def test_builder_matches_reference_fixtures(golden_dir):
    z = np.load(golden_dir / "block_column_cases.npz")
    for i in range(int(z["n_builder"])):
        nrow, ncol, brow, bcol, perm, seed, nnzb = (int(v) for v in z[f"b{i}_args"])
        m = sb.BlockwiseSpMatrix().init_random(nrow, ncol, brow, bcol, float(z[f"b{i}_density_req"]), bool(perm), seed,
                                              values="uniform")
        assert m.nnzb == nnzb and m.density == float(z[f"b{i}_density"])
        assert np.array_equal(m.indptr, z[f"b{i}_indptr"]) and np.array_equal(m.indices, z[f"b{i}_indices"])
        assert m.config_str == z[f"b{i}_config_str"].tobytes().decode()
        if perm:
            assert np.array_equal(m.row_permute_ids, z[f"b{i}_perm"])


def test_bad_block_column_inputs_are_rejected():
    with pytest.raises(sb.ShflbwError):
        sb.BlockwiseSpMatrix().init_random(64, 65, 32, 2, 0.5, False, 1)          # ncol % bcol != 0
    with pytest.raises(sb.ShflbwError):                                           # index 2 is past ncol / bcol
        sb.BlockwiseSpMatrix.from_arrays(2, 4, 2, [0, 1], [2], np.zeros(8, np.float16), bcol=2)
    with pytest.raises(sb.ShflbwError):                                           # values sized for bcol = 1
        sb.BlockwiseSpMatrix.from_arrays(2, 4, 2, [0, 1], [1], np.zeros(2, np.float16), bcol=2)


def _spmm_case(z, i):
    M, K, N, V, bcol, perm, seed = (int(v) for v in z[f"s{i}_args"])
    indptr, indices = z[f"s{i}_indptr"], z[f"s{i}_indices"]
    beta = float(z[f"s{i}_beta"])
    return dict(M=M, K=K, N=N, V=V, bcol=bcol, beta=beta, indptr=indptr, indices=indices,
                perm=z[f"s{i}_perm"] if perm else None, vals=sb.uniform_half(seed, indices.size * V * bcol),
                B=sb.uniform_half(seed + 1000, K * N).reshape(K, N),
                C=sb.uniform_half(seed + 2000, M * N).reshape(M, N) if beta else None, D=z[f"s{i}_D"])


def _conv_case(z, i):
    Bn, H, W, Cc, F, R, S, st, V, bcol, perm, seed = (int(v) for v in z[f"v{i}_args"])
    indptr, indices = z[f"v{i}_indptr"], z[f"v{i}_indices"]
    return dict(Bn=Bn, H=H, W=W, C=Cc, F=F, R=R, S=S, stride=st, V=V, bcol=bcol, indptr=indptr, indices=indices,
                perm=z[f"v{i}_perm"] if perm else None, vals=sb.uniform_half(seed, indices.size * V * bcol),
                x=sb.uniform_half(seed + 1000, Cc * H * W * Bn).reshape(Cc, H, W, Bn), O=z[f"v{i}_O"])


def test_oracle_expansion_matches_reference_host_references(golden_dir):
    """orc_expand_block_columns + the brow x 1 oracle == the reference's get_host_reference with
    bcol > 1, bit for bit (same order of the fp32 additions)."""
    z = np.load(golden_dir / "block_column_cases.npz")
    for i in range(int(z["n_spmm"])):
        c = _spmm_case(z, i)
        ip, ix, v = oa.expand_block_columns(c["V"], c["bcol"], c["indptr"], c["indices"], c["vals"])
        D = oa.spmm_ref(c["M"], c["N"], c["V"], ip, ix, v, c["perm"], c["B"], 1.0, c["C"], c["beta"], threads=4)
        assert np.array_equal(D, c["D"]), f"spmm case {i}"
    for i in range(int(z["n_spconv"])):
        c = _conv_case(z, i)
        ip, ix, v = oa.expand_block_columns(c["V"], c["bcol"], c["indptr"], c["indices"], c["vals"])
        O = oa.spconv_ref_chwn(c["Bn"], c["H"], c["W"], c["C"], c["F"], c["R"], c["S"], c["stride"], c["V"], ip, ix, v,
                               c["perm"], c["x"], threads=4)
        assert np.array_equal(O, c["O"]), f"conv case {i}"


@pytest.mark.skipif(oa.ref_host() is None, reason="oracle/_ref not built (no reference checkout)")
def test_oracle_expansion_matches_reference_run_here():
    r = oa.RefMatrix.init_random(192, 320, 32, 0.3, True, 31, bcol=5)
    vals = sb.uniform_half(31, r.nnzb * 32 * 5)
    B = sb.uniform_half(32, 320 * 16).reshape(320, 16)
    want = oa.ref_spmm_host_reference(192, 320, 16, 32, r.indptr, r.indices, vals, r.perm, B, bcol=5)
    ip, ix, v = oa.expand_block_columns(32, 5, r.indptr, r.indices, vals)
    assert np.array_equal(oa.spmm_ref(192, 16, 32, ip, ix, v, r.perm, B), want)


# ------------------------------------------------------------------------------ GPU --

@pytest.mark.gpu
def test_spmm_on_gpu_matches_reference_fixtures(golden_dir):
    from gpu_util import run_spmm
    z = np.load(golden_dir / "block_column_cases.npz")
    for i in range(int(z["n_spmm"])):
        c = _spmm_case(z, i)
        m = sb.BlockwiseSpMatrix.from_arrays(c["M"], c["K"], c["V"], c["indptr"], c["indices"], c["vals"], c["perm"],
                                             bcol=c["bcol"])
        D, op = run_spmm(m, c["N"], c["B"], 1.0, c["C"], c["beta"])
        assert op._state.kernel == sb.KERNEL_TCGEN05
        assert_close_fp16(D, c["D"], what=f"bcol fixture {i}")


@pytest.mark.gpu
@pytest.mark.parametrize("V,bcol,tokens", [(64, 2, 1024), (64, 4, 256), (128, 2, 512), (32, 8, 256), (16, 4, 128)])
def test_spmm_on_gpu_matches_oracle(V, bcol, tokens):
    from gpu_util import run_spmm
    M, K = 1024, 2048
    m = sb.BlockwiseSpMatrix().init_random(M, K, V, bcol, 0.1, True, 77, values="uniform")
    B = sb.uniform_half(78, K * tokens).reshape(K, tokens)
    D, _ = run_spmm(m, tokens, B)
    ip, ix, v = oa.expand_block_columns(V, bcol, m.indptr, m.indices, m.values)
    assert_close_fp16(D, oa.spmm_ref(M, tokens, V, ip, ix, v, m.row_permute_ids, B), what=f"V={V} bcol={bcol}")
    # every kernel choice reads the same device image
    for kernel in (sb.KERNEL_SIMT,):
        D2, _ = run_spmm(m, tokens, B, kernel=kernel)
        assert_close_fp16(D2, D.astype(np.float32), what="simt vs tcgen05")


@pytest.mark.gpu
def test_spconv_on_gpu_matches_reference_fixtures(golden_dir):
    from gpu_util import run_spconv
    z = np.load(golden_dir / "block_column_cases.npz")
    ran = 0
    for i in range(int(z["n_spconv"])):
        c = _conv_case(z, i)
        if c["C"] % 8:          # NHWC rows of 16 bytes
            continue
        f = sb.BlockwiseSpFilter.from_arrays(c["F"], c["R"], c["S"], c["C"], c["V"], c["indptr"], c["indices"], c["vals"],
                                             c["perm"], bcol=c["bcol"])
        x_nhwc = np.ascontiguousarray(c["x"].transpose(3, 1, 2, 0))
        O, _ = run_spconv(f, c["Bn"], c["H"], c["W"], c["stride"], x_nhwc)
        assert_close_fp16(O, c["O"].transpose(3, 1, 2, 0), what=f"bcol conv fixture {i}")
        ran += 1
    assert ran >= 2


@pytest.mark.gpu
def test_spconv_on_gpu_matches_oracle():
    from gpu_util import run_spconv
    Bn, H, W, Cc, F, V, bcol = 8, 14, 14, 64, 256, 64, 4
    f = sb.BlockwiseSpFilter().init_random(F, 3, 3, Cc, V, bcol, 0.2, True, 5, values="uniform")
    x = sb.uniform_half(6, Bn * H * W * Cc).reshape(Bn, H, W, Cc)
    O, _ = run_spconv(f, Bn, H, W, 1, x)
    ip, ix, v = oa.expand_block_columns(V, bcol, f.indptr, f.indices, f.values)
    assert_close_fp16(O, oa.spconv_ref_nhwc(Bn, H, W, Cc, F, 3, 3, 1, V, ip, ix, v, f.row_permute_ids, x), what="bcol conv")
