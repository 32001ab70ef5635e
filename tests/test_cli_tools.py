"""The command-line benchmarks: same flags and output line as the reference's
benchmark.spmm.out / benchmark.spconv.out (block_sparse/benchmark/benchmark.spmm.cu:96-107,
benchmark.spconv.cu:104-115, flags block_sparse/benchmark/argparse_util.h:10-119, 121-264)."""
import subprocess

import pytest

from shflbw_sparse_nn_b200.build import build_tools


@pytest.fixture(scope="module")
def tools():
    return build_tools()


def test_tools_build_and_refuse_incomplete_arguments(tools):
    for name in ("benchmark.spmm.out", "benchmark.spconv.out"):
        res = subprocess.run([str(tools[name]), "--d", "0.1"], capture_output=True, text=True)
        assert res.returncode != 0
        assert "Required cmdline args" in res.stderr and "density" in res.stderr
    res = subprocess.run([str(tools["benchmark.spmm.out"]), "--m", "64", "--n", "64", "--k", "64", "--d", "0.5",
                          "--sparsity-type", "block", "--block-size", "48"], capture_output=True, text=True)
    assert res.returncode != 0 and "Unsupported block size" in res.stderr


@pytest.mark.gpu
def test_spmm_tool_prints_the_reference_line_and_round_trips_a_pattern(tools, tmp_path):
    pat = tmp_path / "pattern.txt"
    base = [str(tools["benchmark.spmm.out"]), "--m", "500", "--n", "1000", "--k", "512", "--d", "0.2",
            "--sparsity-type", "block", "--block-size", "64", "--row-permute"]
    res = subprocess.run(base + ["--store-pattern", str(pat)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert "m padded to : 512" in res.stderr and "n padded to : 1024" in res.stderr
    f = res.stdout.split()
    # GPU_CC <config_str: 7 fields> n BLOCK_SZ BN BK WM WN WK MMA_M MMA_N MMA_K NSTAGE t (us) x (effective tflop/s)
    assert len(f) == 1 + 7 + 1 + 10 + 5
    assert f[0] == "100" and f[1:5] == ["512", "512", "64", "1"] and f[7] == "row-permute"
    assert f[8] == "1024" and f[9] == "64" and f[-4] == "(us)" and f[-2:] == ["(effective", "tflop/s)"]
    t_us, tflops = float(f[-5]), float(f[-3])
    assert t_us > 0 and abs(tflops - 2 * 512 * 1024 * 512 / 1e9 / (t_us / 1e3)) < 1e-2 * tflops
    res2 = subprocess.run([str(tools["benchmark.spmm.out"]), "--m", "1", "--n", "1000", "--k", "1", "--d", "0.2",
                           "--sparsity-type", "block", "--block-size", "64", "--load-pattern", str(pat)],
                          capture_output=True, text=True)
    assert res2.returncode == 0, res2.stderr
    g = res2.stdout.split()
    assert g[1:6] == f[1:6] and g[7] == f[7]        # same shape, achieved density and permutation flag (the text format carries no seed)


@pytest.mark.gpu
def test_spconv_tool_prints_the_reference_line(tools):
    res = subprocess.run([str(tools["benchmark.spconv.out"]), "--B", "8", "--H", "7", "--W", "7", "--C", "64", "--F", "100",
                          "--R", "3", "--S", "3", "--stride", "2", "--d", "0.25", "--sparsity-type", "block",
                          "--block-size", "32", "--row-permute"], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert "F padded to : 128" in res.stderr
    f = res.stdout.split()
    # GPU_CC <config_str: 9 fields> B H W stride BLOCK_SZ BN BK WM WN WK MMA_M MMA_N MMA_K NSTAGE t (us) x (effective tflop/s)
    assert len(f) == 1 + 9 + 4 + 10 + 5
    assert f[0] == "100" and f[1:7] == ["128", "3", "3", "64", "32", "1"] and f[9] == "filter-permute"
    assert f[10:14] == ["8", "7", "7", "2"] and f[14] == "32" and float(f[-5]) > 0 and f[-4] == "(us)"
