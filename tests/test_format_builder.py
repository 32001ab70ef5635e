"""The product's host format code (builder, dump/load, validation, device images) against
the oracle and the committed reference fixtures.  Bit-exact bar: integer/index work."""
import ctypes
import hashlib
import json

import numpy as np
import pytest

import oracle_api as oa
import shflbw_sparse_nn_b200 as sb
from shflbw_sparse_nn_b200 import _cabi


def test_builder_reproduces_reference_golden_dump(golden_dir):
    pin = json.loads((golden_dir / "mtx_dump_pin.json").read_text())
    ctypes.CDLL(None).srand(1)  # libc stream of a fresh process
    m = sb.BlockwiseSpMatrix().init_random(1024, 1024, 32, 1, 0.2, False, 2021)
    text = m.dump()
    assert len(text) == pin["size"] and hashlib.sha256(text).hexdigest() == pin["sha256"]
    assert m.nnzb == int(pin["head_lines"][2])
    # load -> dump is the identity on the reference's text
    again = sb.BlockwiseSpMatrix().load(text)
    assert again.dump() == text
    assert np.array_equal(again.indices, m.indices) and np.array_equal(again.values, m.values)


def test_builder_matches_reference_fixture_grid(golden_dir):
    z = np.load(golden_dir / "builder_cases.npz")
    for i in range(int(z["n_cases"])):
        nrow, ncol, brow, perm, seed, nnzb = (int(v) for v in z[f"c{i}_args"])
        m = sb.BlockwiseSpMatrix().init_random(nrow, ncol, brow, 1, float(z[f"c{i}_density_req"]), bool(perm),
                                              seed, values="uniform")
        assert m.nnzb == nnzb
        assert np.array_equal(m.indptr, z[f"c{i}_indptr"])
        assert hashlib.sha256(m.indices.tobytes()).digest() == z[f"c{i}_indices_sha"].tobytes()
        assert m.density == float(z[f"c{i}_density"])
        assert m.config_str == z[f"c{i}_config_str"].tobytes().decode()
        if perm:
            assert hashlib.sha256(m.row_permute_ids.tobytes()).digest() == z[f"c{i}_perm_sha"].tobytes()
        else:
            assert m.row_permute_ids.size == 0
        m.validate()
    f = sb.BlockwiseSpFilter().init_random(2048, 3, 3, 512, 64, 1, 0.1, True, 2021, values="uniform")
    assert f.config_str == z["filter_config_str"].tobytes().decode()
    assert (f.F, f.R, f.S, f.C) == (2048, 3, 3, 512) and f.ncol == 4608


@pytest.mark.parametrize("nrow,ncol,brow,d,perm,seed", [(256, 256, 32, 0.1, True, 2021), (512, 320, 64, 0.23, False, 5),
                                                        (384, 128, 128, 0.5, True, 77), (64, 1024, 16, 0.03, True, 2)])
def test_builder_matches_oracle(nrow, ncol, brow, d, perm, seed):
    n, indptr, indices = oa.random_mask(nrow, ncol, brow, 1, d, seed)
    oa.srand(123)
    vals = oa.fill_int9(n * brow)
    oa.srand(123)
    m = sb.BlockwiseSpMatrix().init_random(nrow, ncol, brow, 1, d, perm, seed, values="int9")
    assert m.nnzb == n and np.array_equal(m.indptr, indptr) and np.array_equal(m.indices, indices)
    assert np.array_equal(m.values.view(np.uint16), vals.view(np.uint16))
    p = oa.row_permutation(nrow, seed) if perm else None
    if perm:
        assert np.array_equal(m.row_permute_ids, p)
    assert m.dump() == oa.dump_text(nrow, ncol, brow, indptr, indices, vals, p)
    assert np.array_equal(m.meta_h, oa.meta_image(indptr, indices, p))


def test_uniform_values_are_the_documented_stream():
    m = sb.BlockwiseSpMatrix().init_random(256, 256, 32, 1, 0.1, True, 2021, values="uniform")
    expect = sb.uniform_half(2021, m.nnzb * 32)
    assert np.array_equal(m.values.view(np.uint16), expect.view(np.uint16))
    assert np.abs(expect.astype(np.float32)).max() <= 1.0
    assert abs(float(expect.astype(np.float32).mean())) < 0.05


def test_from_arrays_roundtrip_and_documented_example():
    # example/spmatrix_dump_load.md, restated with bcol = 1 (2 columns per row block)
    indptr, indices = np.array([0, 2, 4], np.int32), np.array([0, 1, 2, 3], np.int32)
    vals = np.array([1, 2, 1, 2, 3, 1, 1, 2], np.float16)
    perm = np.array([0, 3, 1, 2], np.int32)
    m = sb.BlockwiseSpMatrix.from_arrays(4, 4, 2, indptr, indices, vals, perm)
    assert m.dump() == oa.dump_text(4, 4, 2, indptr, indices, vals, perm)
    m2 = sb.BlockwiseSpMatrix().load(m.dump())
    assert m2.row_permute and np.array_equal(m2.row_permute_ids, perm) and np.array_equal(m2.values, vals)


def test_malformed_inputs_are_rejected_not_aborted():
    ok_ptr, ok_idx = np.array([0, 2, 3], np.int32), np.array([1, 5, 0], np.int32)
    vals = np.zeros(3 * 2, np.float16)
    bad = [
        (np.array([0, 2, 4], np.int32), ok_idx, None),            # indptr end != nnzb
        (np.array([0, 3, 2], np.int32), ok_idx, None),            # not monotone
        (ok_ptr, np.array([5, 1, 0], np.int32), None),            # not ascending inside a block
        (ok_ptr, np.array([1, 8, 0], np.int32), None),            # column out of range
        (ok_ptr, np.array([1, 1, 0], np.int32), None),            # duplicate column
        (ok_ptr, ok_idx, np.array([0, 1, 1, 3], np.int32)),       # perm not a permutation
        (ok_ptr, ok_idx, np.array([0, 1, 2, 4], np.int32)),       # perm out of range
    ]
    for ptr, idx, perm in bad:
        with pytest.raises(sb.ShflbwError) as e:
            sb.BlockwiseSpMatrix.from_arrays(4, 8, 2, ptr, idx, vals, perm)
        assert e.value.status == _cabi.ERR_BAD_FORMAT
    with pytest.raises(sb.ShflbwError):
        sb.BlockwiseSpMatrix().init_random(100, 64, 32, 1, 0.1, False, 1)   # nrow % brow != 0
    with pytest.raises(sb.ShflbwError):
        sb.BlockwiseSpMatrix().init_random(64, 63, 32, 2, 0.1, False, 1)    # ncol % bcol != 0
    with pytest.raises(sb.ShflbwError):
        sb.BlockwiseSpMatrix().load(b"4 4 2 2 1 0 0 1")                     # truncated text
    sb.BlockwiseSpMatrix.from_arrays(4, 8, 2, ok_ptr, ok_idx, vals, None)   # the good one passes


def test_empty_and_ragged_row_blocks():
    # block 0 empty, block 1 one column, block 2 seventeen columns (one over a K-step)
    indptr = np.array([0, 0, 1, 18], np.int32)
    indices = np.concatenate([[3], np.arange(17)]).astype(np.int32)
    vals = sb.uniform_half(1, 18 * 32)
    m = sb.BlockwiseSpMatrix.from_arrays(96, 32, 32, indptr, indices, vals)
    assert m.nnzb == 18 and list(np.diff(m.indptr)) == [0, 1, 17]
    meta = m.meta_h
    assert meta.size == 8 + 24 + 0 and np.array_equal(meta[:4], indptr) and np.array_equal(meta[8:26], indices)


def test_fold_input_order_relabels_channels_and_keeps_the_format_invariants():
    """shflbw_filter_fold_input_order: column (r, s, c) moves to (r, s, stored position of c in the
    producer); lists stay sorted, values follow their columns, the filter's own permutation stays."""
    prod = sb.BlockwiseSpFilter().init_random(64, 1, 1, 16, 32, 1, 0.5, True, 3, values="uniform")
    f = sb.BlockwiseSpFilter().init_random(96, 3, 3, 64, 32, 1, 0.2, True, 4, values="uniform")
    g = f.fold_input_order(prod)
    g.validate()
    assert (g.F, g.R, g.S, g.C, g.nnzb, g.brow) == (f.F, f.R, f.S, f.C, f.nnzb, f.brow)
    assert np.array_equal(g.indptr, f.indptr) and np.array_equal(g.row_permute_ids, f.row_permute_ids)

    def dense(m):
        d = np.zeros((m.nrow, m.ncol), np.uint16)
        v = m.values.reshape(-1, m.brow)
        for i in range(m.nrow // m.brow):
            for p in range(m.indptr[i], m.indptr[i + 1]):
                d[i * m.brow:(i + 1) * m.brow, m.indices[p]] = v[p]
        return d

    where = np.empty(64, np.int64)
    where[prod.row_permute_ids] = np.arange(64)          # logical channel -> stored position
    cols = (np.arange(f.ncol) // 64) * 64 + where[np.arange(f.ncol) % 64]
    want = np.zeros_like(dense(f))
    want[:, cols] = dense(f)
    assert np.array_equal(dense(g), want)
    for i in range(g.nrow // g.brow):
        assert np.all(np.diff(g.indices[g.indptr[i]:g.indptr[i + 1]]) > 0)
    # a producer without a permutation folds to the identity
    ident = sb.BlockwiseSpFilter().init_random(64, 1, 1, 16, 32, 1, 0.5, False, 3, values="uniform")
    h = f.fold_input_order(ident)
    assert np.array_equal(h.indices, f.indices) and np.array_equal(h.values, f.values)
