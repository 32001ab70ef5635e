"""Generates the committed fixtures in this folder by running the UNMODIFIED reference
(compiled from its own sources into oracle/_ref/ by oracle/Makefile).  Needs the reference
checkout; the tests only need the files written here.

    make -C oracle && python tests/golden/make_golden.py

Writes:
  mtx_dump_pin.json       SHA-256, size and leading fields of the reference's own golden file
                          example/mtx_dump.txt, plus the same for a dump re-created by
                          init_random(1024,1024,32,1,0.2,false,2021) in a fresh process
  builder_cases.npz       mask / permutation / achieved density / config string produced by the
                          reference builder for a grid of (shape, V, density, permute, seed)
  spmm_cases.npz          reference get_host_reference outputs (fp32) on small seeded inputs
  spconv_cases.npz        reference conv get_host_reference outputs (fp32), reference layouts
  block_column_cases.npz  the same three kinds of output for brow x bcol blocks with bcol > 1
                          (`python tests/golden/make_golden.py blocks` writes this file alone)
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

import oracle_api as oa  # noqa: E402
from shflbw_sparse_nn_b200.blockwise import uniform_half  # noqa: E402

import os  # noqa: E402

# checkout of the reference project (same default as oracle/Makefile's REF: a sibling of this repository)
REF_GOLDEN = Path(os.environ.get("REF", str(HERE.parent.parent.parent / "reference"))) / "example" / "mtx_dump.txt"

BUILDER_GRID = [
    # nrow, ncol, brow, density, permute, seed
    (256, 256, 32, 0.1, True, 2021),     # small correctness case (V=32)
    (1024, 1024, 32, 0.2, False, 2021),  # the reference's example / golden dump
    (1024, 1024, 16, 0.1, True, 2021),   # reference test shape, V=16
    (1024, 1024, 64, 0.1, True, 2021),
    (1024, 1024, 128, 0.1, False, 2021),
    (4096, 4096, 64, 0.1, True, 2021),   # headline SpMM shape
    (2048, 4608, 64, 0.1, True, 2021),   # headline SpConv filter matrix (2048 x 3*3*512)
    (768, 3072, 128, 0.05, True, 7),
    (64, 64, 64, 0.2, True, 3),          # single row block, K smaller than one stage
    (128, 96, 32, 0.5, False, 11),
]


def write_block_column_cases() -> None:
    """bcol > 1: the reference's builder and both of its host references."""
    z = {}
    grid = [  # nrow, ncol, brow, bcol, density, permute, seed
        (256, 256, 32, 2, 0.1, True, 2021),
        (512, 384, 64, 4, 0.2, False, 5),
        (128, 1024, 16, 8, 0.15, True, 9),
    ]
    for i, (nrow, ncol, brow, bcol, d, perm, seed) in enumerate(grid):
        r = oa.RefMatrix.init_random(nrow, ncol, brow, d, perm, seed, bcol=bcol)
        z[f"b{i}_args"] = np.array([nrow, ncol, brow, bcol, int(perm), seed, r.nnzb], np.int64)
        z[f"b{i}_density_req"], z[f"b{i}_density"] = np.float32(d), np.float32(r.density)
        z[f"b{i}_indptr"], z[f"b{i}_indices"] = r.indptr, r.indices
        if perm:
            z[f"b{i}_perm"] = r.perm
        z[f"b{i}_config_str"] = np.frombuffer(r.config_str.encode(), np.uint8)
    z["n_builder"] = np.int64(len(grid))
    cases = [  # M, K, N, V, bcol, density, permute, seed, beta
        (128, 256, 40, 32, 2, 0.2, True, 11, 0.0),
        (256, 192, 64, 64, 4, 0.25, True, 12, 1.0),
        (64, 128, 24, 16, 8, 0.3, False, 13, 0.0),
    ]
    for i, (M, K, N, V, bcol, d, perm, seed, beta) in enumerate(cases):
        r = oa.RefMatrix.init_random(M, K, V, d, perm, seed, bcol=bcol)
        vals = uniform_half(seed, r.nnzb * V * bcol)
        B = uniform_half(seed + 1000, K * N).reshape(K, N)
        Cm = uniform_half(seed + 2000, M * N).reshape(M, N) if beta != 0.0 else None
        D = oa.ref_spmm_host_reference(M, K, N, V, r.indptr, r.indices, vals, r.perm, B, 1.0, Cm, beta, bcol=bcol)
        z[f"s{i}_args"] = np.array([M, K, N, V, bcol, int(perm), seed], np.int64)
        z[f"s{i}_beta"] = np.float32(beta)
        z[f"s{i}_indptr"], z[f"s{i}_indices"] = r.indptr, r.indices
        if perm:
            z[f"s{i}_perm"] = r.perm
        z[f"s{i}_D"] = D
    z["n_spmm"] = np.int64(len(cases))
    ccases = [  # B, H, W, C, F, R, S, stride, V, bcol, density, permute, seed
        (8, 6, 6, 16, 64, 3, 3, 1, 32, 2, 0.2, True, 21),
        (8, 5, 7, 24, 128, 3, 3, 1, 64, 4, 0.3, False, 22),   # C % bcol == 0, blocks stay inside a tap
        (8, 4, 4, 9, 64, 1, 1, 1, 32, 3, 0.5, True, 23),
    ]
    for i, (Bn, H, W, Cc, F, R, S, st, V, bcol, d, perm, seed) in enumerate(ccases):
        r = oa.RefMatrix.filter_init_random(F, R, S, Cc, V, d, perm, seed, bcol=bcol)
        vals = uniform_half(seed, r.nnzb * V * bcol)
        x = uniform_half(seed + 1000, Cc * H * W * Bn).reshape(Cc, H, W, Bn)
        O = oa.ref_spconv_host_reference(Bn, H, W, Cc, F, R, S, st, V, r.indptr, r.indices, vals, r.perm, x, bcol=bcol)
        z[f"v{i}_args"] = np.array([Bn, H, W, Cc, F, R, S, st, V, bcol, int(perm), seed], np.int64)
        z[f"v{i}_indptr"], z[f"v{i}_indices"] = r.indptr, r.indices
        if perm:
            z[f"v{i}_perm"] = r.perm
        z[f"v{i}_O"] = O
    z["n_spconv"] = np.int64(len(ccases))
    np.savez_compressed(HERE / "block_column_cases.npz", **z)


def main() -> None:
    assert oa.ref_host() is not None, "build oracle/_ref first (make -C oracle)"
    if sys.argv[1:] == ["blocks"]:
        write_block_column_cases()
        return
    # -- 1. the reference's own golden file --------------------------------------------
    gold = REF_GOLDEN.read_bytes()
    m = oa.RefMatrix.init_random(1024, 1024, 32, 0.2, False, 2021)  # first rand() consumer here
    redump = m.dump()
    lines = gold.split(b"\n")
    pin = {
        "source": "example/mtx_dump.txt of the reference",
        "call": "init_random(1024,1024,32,1,0.2,false,2021) as first rand() consumer, then dump()",
        "size": len(gold),
        "sha256": hashlib.sha256(gold).hexdigest(),
        "head_lines": [l.decode() for l in lines[:6]],
        "indptr_line": lines[6].decode(),
        "indices_first_32": lines[7].decode().split()[:32],
        "values_first_64": lines[8].decode().split()[:64],
        "reference_rebuild_identical": redump == gold,
    }
    (HERE / "mtx_dump_pin.json").write_text(json.dumps(pin, indent=1) + "\n")

    # -- 2. builder grid ---------------------------------------------------------------
    out = {}
    for i, (nrow, ncol, brow, d, perm, seed) in enumerate(BUILDER_GRID):
        r = oa.RefMatrix.init_random(nrow, ncol, brow, d, perm, seed)
        out[f"c{i}_args"] = np.array([nrow, ncol, brow, int(perm), seed, r.nnzb], np.int64)
        out[f"c{i}_density_req"] = np.float32(d)
        out[f"c{i}_density"] = np.float32(r.density)
        out[f"c{i}_indptr"] = r.indptr
        out[f"c{i}_indices_sha"] = np.frombuffer(hashlib.sha256(r.indices.tobytes()).digest(), np.uint8)
        out[f"c{i}_indices_head"] = r.indices[:64]
        if perm:
            out[f"c{i}_perm_sha"] = np.frombuffer(hashlib.sha256(r.perm.tobytes()).digest(), np.uint8)
            out[f"c{i}_perm_head"] = r.perm[:64]
        out[f"c{i}_config_str"] = np.frombuffer(r.config_str.encode(), np.uint8)
    f = oa.RefMatrix.filter_init_random(2048, 3, 3, 512, 64, 0.1, True, 2021)
    out["filter_config_str"] = np.frombuffer(f.config_str.encode(), np.uint8)
    out["n_cases"] = np.int64(len(BUILDER_GRID))
    np.savez_compressed(HERE / "builder_cases.npz", **out)

    # -- 3. SpMM CPU reference outputs ------------------------------------------------------
    sp = {}
    cases = [  # M, K, N, V, density, permute, seed, beta
        (256, 256, 64, 32, 0.1, True, 2021, 0.0),   # config 1 with a 64-column slice of B
        (128, 192, 40, 64, 0.2, True, 5, 1.0),      # N % 16 != 0, beta = 1 as the reference example
        (256, 128, 24, 128, 0.3, False, 9, 0.0),
    ]
    for i, (M, K, N, V, d, perm, seed, beta) in enumerate(cases):
        r = oa.RefMatrix.init_random(M, K, V, d, perm, seed)
        vals = uniform_half(seed, r.nnzb * V)
        B = uniform_half(seed + 1000, K * N).reshape(K, N)
        Cm = uniform_half(seed + 2000, M * N).reshape(M, N) if beta != 0.0 else None
        D = oa.ref_spmm_host_reference(M, K, N, V, r.indptr, r.indices, vals, r.perm, B, 1.0, Cm, beta)
        sp[f"s{i}_args"] = np.array([M, K, N, V, int(perm), seed], np.int64)
        sp[f"s{i}_beta"] = np.float32(beta)
        sp[f"s{i}_density"] = np.float32(d)
        sp[f"s{i}_indptr"], sp[f"s{i}_indices"] = r.indptr, r.indices
        if perm:
            sp[f"s{i}_perm"] = r.perm
        sp[f"s{i}_D"] = D
    sp["n_cases"] = np.int64(len(cases))
    np.savez_compressed(HERE / "spmm_cases.npz", **sp)

    # -- 4. SpConv CPU reference outputs (reference layouts: in [C][H][W][B], out [F][H][W][B]) --
    cv = {}
    ccases = [  # B, H, W, C, F, R, S, stride, V, density, permute, seed
        (8, 6, 6, 16, 64, 3, 3, 1, 32, 0.2, True, 2021),
        (8, 6, 6, 16, 64, 3, 3, 2, 32, 0.2, False, 2021),
        (8, 5, 7, 32, 128, 1, 1, 1, 64, 0.3, True, 4),
    ]
    for i, (Bn, H, W, Cc, F, R, S, st, V, d, perm, seed) in enumerate(ccases):
        r = oa.RefMatrix.filter_init_random(F, R, S, Cc, V, d, perm, seed)
        vals = uniform_half(seed, r.nnzb * V)
        x = uniform_half(seed + 1000, Cc * H * W * Bn).reshape(Cc, H, W, Bn)
        O = oa.ref_spconv_host_reference(Bn, H, W, Cc, F, R, S, st, V, r.indptr, r.indices, vals, r.perm, x)
        cv[f"v{i}_args"] = np.array([Bn, H, W, Cc, F, R, S, st, V, int(perm), seed], np.int64)
        cv[f"v{i}_density"] = np.float32(d)
        cv[f"v{i}_indptr"], cv[f"v{i}_indices"] = r.indptr, r.indices
        if perm:
            cv[f"v{i}_perm"] = r.perm
        cv[f"v{i}_O"] = O
    cv["n_cases"] = np.int64(len(ccases))
    np.savez_compressed(HERE / "spconv_cases.npz", **cv)
    write_block_column_cases()
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
