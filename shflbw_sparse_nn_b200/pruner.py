"""Dense weights -> Shfl-BW: choose a row permutation and per-block column sets for a given
density, then hand the arrays to the format builder.

The reference only ever builds RANDOM patterns (`BlockwiseSpMatrix::init_random`,
block_sparse/spmm/blockwise_format.h:70-123); its README points to the paper for how real
weights are pruned: rows that want to keep similar columns are shuffled into the same V-row
block, and each block keeps the columns that matter most to its rows.  This module is a small,
deterministic restatement of that idea for users who arrive with a trained layer:

    m, info = prune_matrix(W, V=64, density=0.1)            # W: [M][K] array-like
    f, info = prune_conv_filter(Wc, V=64, density=0.2)      # Wc: [F][C][R][S] (PyTorch order)

`m` / `f` are ordinary `BlockwiseSpMatrix` / `BlockwiseSpFilter` objects (dump, to device, SpMM,
SpConv as usual); `info["retained"]` is the fraction of the squared weight mass kept.

Algorithm (all on the host, numpy):
  1. every row gets a signature: its squared weights;
  2. balanced clustering into M/V groups of exactly V rows: start from the identity grouping (or
     a seeded random one), then repeat {score each group's columns by the summed signatures of
     its rows; mark each group's top-n columns; reassign rows, most decided first, to the group
     whose marked columns hold most of the row's mass and that still has room};
  3. each group keeps the n = round(density * K) columns with the largest summed signature,
     ascending (the format's invariant); values are the original weights, rounded to fp16.
With permute=False step 2 is skipped (plain vector-wise block pruning of consecutive rows)."""
from __future__ import annotations

import numpy as np

from .blockwise import BlockwiseSpFilter, BlockwiseSpMatrix


def _as_f32(a) -> np.ndarray:
    if hasattr(a, "detach"):          # torch.Tensor without importing torch here
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _top_mask(scores: np.ndarray, n: int) -> np.ndarray:
    """Boolean mask of the n largest entries of every row of `scores` (ties: lower index first)."""
    X, K = scores.shape
    order = np.argsort(-scores, axis=1, kind="stable")[:, :n]
    mask = np.zeros((X, K), dtype=bool)
    np.put_along_axis(mask, order, True, axis=1)
    return mask


def group_rows(sig: np.ndarray, V: int, n_keep: int, iters: int = 8, seed: int | None = None) -> np.ndarray:
    """Balanced grouping of the rows of `sig` ([M][K], non-negative) into M/V groups of V rows.
    Returns `group_of_row` ([M] ints).  Deterministic for a given seed (None: start from the
    identity grouping)."""
    M, K = sig.shape
    X = M // V
    if seed is None:
        group = np.repeat(np.arange(X), V)
    else:
        group = np.repeat(np.arange(X), V)[np.random.default_rng(seed).permutation(M)]
    if X == 1:
        return group
    for _ in range(iters):
        centre = np.zeros((X, K), dtype=np.float64)
        np.add.at(centre, group, sig)
        marked = _top_mask(centre, n_keep).astype(np.float32)           # [X][K]
        gain = sig @ marked.T                                            # [M][X]: row mass inside each group's columns
        best2 = np.partition(gain, X - 2, axis=1)[:, X - 2:]             # two largest per row
        order = np.argsort(-(best2[:, 1] - best2[:, 0]), kind="stable")  # most decided rows first
        room = np.full(X, V)
        new_group = np.empty(M, dtype=np.int64)
        pref = np.argsort(-gain, axis=1, kind="stable")
        for r in order:
            for g in pref[r]:
                if room[g]:
                    new_group[r] = g
                    room[g] -= 1
                    break
        if np.array_equal(new_group, group):
            break
        group = new_group
    return group


def prune_matrix(weight, V: int, density: float, permute: bool = True, iters: int = 8, seed: int | None = None):
    """[M][K] dense weights -> (BlockwiseSpMatrix, info).  M % V == 0; 0 < density <= 1."""
    W = _as_f32(weight)
    if W.ndim != 2:
        raise ValueError("weight must be a matrix [M][K]")
    M, K = W.shape
    if M % V:
        raise ValueError(f"M = {M} is not a multiple of the block height V = {V}")
    if not 0.0 < density <= 1.0:
        raise ValueError("density must be in (0, 1]")
    X = M // V
    n_keep = max(1, min(K, int(round(density * K))))
    sig = W * W
    group = group_rows(sig, V, n_keep, iters, seed) if permute else np.repeat(np.arange(X), V)
    # stored row p = g*V + j holds original row rows_of[g][j]; row_permute_ids[p] = that original row
    stored = np.argsort(group, kind="stable")
    centre = np.zeros((X, K), dtype=np.float64)
    np.add.at(centre, group, sig)
    cols = np.sort(np.argsort(-centre, axis=1, kind="stable")[:, :n_keep], axis=1)     # [X][n_keep] ascending
    indptr = (np.arange(X + 1) * n_keep).astype(np.int32)
    indices = cols.reshape(-1).astype(np.int32)
    Wp = W[stored].reshape(X, V, K)                                                    # stored order
    vals = np.take_along_axis(Wp, cols[:, None, :], axis=2)                            # [X][V][n_keep]
    values = np.ascontiguousarray(vals.transpose(0, 2, 1)).astype(np.float16).reshape(-1)   # values[p*V + m]
    perm = stored.astype(np.int32) if permute else None
    m = BlockwiseSpMatrix.from_arrays(M, K, V, indptr, indices, values.view(np.uint16), perm)
    kept = float((vals.astype(np.float64) ** 2).sum())
    info = {"retained": kept / max(float(sig.sum(dtype=np.float64)), 1e-300), "columns_per_block": n_keep,
            "density": n_keep / K, "group_of_row": group}
    return m, info


def prune_conv_filter(weight, V: int, density: float, permute: bool = True, iters: int = 8, seed: int | None = None):
    """[F][C][R][S] conv weights (PyTorch layout) -> (BlockwiseSpFilter, info).  The filter matrix
    is F x (R*S*C) with column k = (r*S + s)*C + c, the layout the SpConv path expects."""
    W = _as_f32(weight)
    if W.ndim != 4:
        raise ValueError("weight must be [F][C][R][S]")
    F, C_, R, S = W.shape
    mat = np.ascontiguousarray(W.transpose(0, 2, 3, 1)).reshape(F, R * S * C_)
    m, info = prune_matrix(mat, V, density, permute, iters, seed)
    f = BlockwiseSpFilter.from_arrays(F, R, S, C_, V, m.indptr, m.indices, m.values,
                                      m.row_permute_ids if permute else None)
    return f, info
