"""Dense weights -> Shfl-BW (shflbw_sparse_nn_b200/pruner.py): the produced object is the masked
dense matrix in the format's layout, and grouping rows with similar column needs keeps more of
the weight mass than pruning consecutive rows.  CPU only; the SpMM check runs on the oracle."""
import numpy as np
import pytest

import oracle_api as oa
from shflbw_sparse_nn_b200.pruner import group_rows, prune_conv_filter, prune_matrix


def _densify(m):
    """Logical dense matrix (rows in ORIGINAL order) of a Shfl-BW object, fp16."""
    d = np.zeros((m.nrow, m.ncol), np.float16)
    v = m.values.reshape(-1, m.brow)
    perm = m.row_permute_ids if m.row_permute else np.arange(m.nrow)
    for i in range(m.nrow // m.brow):
        rows = perm[i * m.brow:(i + 1) * m.brow]
        for p in range(m.indptr[i], m.indptr[i + 1]):
            d[rows, m.indices[p]] = v[p]
    return d


def _planted(M, K, V, n_keep, seed):
    """Rows drawn from M/V prototypes, each prototype using its own n_keep columns; rows shuffled."""
    rng = np.random.default_rng(seed)
    X = M // V
    W = rng.normal(0, 0.01, (M, K)).astype(np.float32)           # small background
    proto = np.repeat(np.arange(X), V)
    for g in range(X):
        cols = rng.choice(K, n_keep, replace=False)
        W[np.ix_(proto == g, cols)] += rng.normal(0, 1.0, (V, n_keep)).astype(np.float32)
    shuffle = rng.permutation(M)
    return W[shuffle], proto[shuffle]


@pytest.mark.parametrize("permute", [False, True])
def test_pruned_object_is_the_masked_dense_matrix(permute):
    rng = np.random.default_rng(5)
    W = rng.normal(size=(128, 96)).astype(np.float32)
    m, info = prune_matrix(W, V=32, density=0.25, permute=permute)
    m.validate()
    assert m.nrow == 128 and m.ncol == 96 and m.brow == 32 and m.nnzb == 4 * 24
    assert bool(m.row_permute) == permute and info["columns_per_block"] == 24
    d = _densify(m)
    kept = d != 0
    assert np.array_equal(d[kept], W.astype(np.float16)[kept])   # kept entries are the original weights
    assert kept.sum(axis=1).max() <= 24 and kept.sum() > 0.9 * 128 * 24
    if permute:
        assert sorted(m.row_permute_ids.tolist()) == list(range(128))
    for i in range(4):                                           # ascending column lists
        assert np.all(np.diff(m.indices[m.indptr[i]:m.indptr[i + 1]]) > 0)
    # retained mass reported = mass of the kept entries
    assert abs(info["retained"] - float((W[kept] ** 2).sum() / (W ** 2).sum())) < 1e-3


def test_row_grouping_recovers_planted_structure_and_beats_consecutive_rows():
    M, K, V, n_keep = 256, 512, 32, 51
    W, proto = _planted(M, K, V, n_keep, seed=11)
    m_perm, info_perm = prune_matrix(W, V, density=0.1, permute=True, seed=3)
    m_cons, info_cons = prune_matrix(W, V, density=0.1, permute=False)
    assert info_perm["retained"] > 0.97                          # every block found its prototype's columns
    assert info_cons["retained"] < 0.5                           # consecutive rows mix prototypes
    g = info_perm["group_of_row"]
    for grp in range(M // V):                                    # groups are pure and full
        members = proto[g == grp]
        assert members.size == V and np.unique(members).size == 1
    assert np.bincount(group_rows(W * W, V, n_keep, seed=None), minlength=M // V).tolist() == [V] * (M // V)


def test_spmm_on_the_pruned_matrix_equals_masked_dense_matmul():
    rng = np.random.default_rng(9)
    W = rng.normal(size=(64, 128)).astype(np.float32)
    m, _ = prune_matrix(W, V=32, density=0.3, permute=True)
    B = rng.uniform(-1, 1, (128, 16)).astype(np.float16)
    ref = oa.spmm_ref(64, 16, 32, m.indptr, m.indices, m.values, m.row_permute_ids, B)
    want = _densify(m).astype(np.float32) @ B.astype(np.float32)
    assert np.allclose(ref, want, rtol=1e-4, atol=1e-4)


def test_conv_filter_layout():
    rng = np.random.default_rng(2)
    Wc = rng.normal(size=(64, 8, 3, 3)).astype(np.float32)        # [F][C][R][S]
    f, info = prune_conv_filter(Wc, V=32, density=0.5, permute=True)
    f.validate()
    assert (f.F, f.R, f.S, f.C) == (64, 3, 3, 8) and f.ncol == 72 and f.nnzb == 2 * 36
    d = _densify(f).reshape(64, 3, 3, 8)                          # [F][r][s][c], k = (r*S + s)*C + c
    kept = d != 0
    assert np.array_equal(d[kept], Wc.transpose(0, 2, 3, 1).astype(np.float16)[kept])
    assert 0.5 < info["retained"] <= 1.0


def test_argument_checks():
    with pytest.raises(ValueError):
        prune_matrix(np.zeros((100, 8), np.float32), V=32, density=0.5)
    with pytest.raises(ValueError):
        prune_matrix(np.zeros((64, 8), np.float32), V=32, density=0.0)
    with pytest.raises(ValueError):
        prune_conv_filter(np.zeros((64, 8), np.float32), V=32, density=0.5)
