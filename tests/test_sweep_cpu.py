"""Host logic of the sweep tool (the reference driver's command line, GEMM/gemm_main.cpp:196-313): arguments,
the 64-cube list, the GFLOPS formula and the CSV lines.  No GPU."""
import importlib.util
import os

import pytest

from __graft_entry__ import PKG_DIR


@pytest.fixture(scope="module")
def sweep():
    spec = importlib.util.spec_from_file_location("tcfp8_sweep", os.path.join(PKG_DIR, "sweep.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_arguments_follow_the_reference_driver(sweep):
    a = sweep.parse("4096 4096 4096 2 0 1 1".split())          # a line of the reference's testbench.sh
    assert (a.dimM, a.dimK, a.dimN, a.kernel, a.verify, a.record, a.testbench) == (4096, 4096, 4096, 2, 0, 1, 1)
    with pytest.raises(SystemExit):
        sweep.parse("128 128 128 10 0 0 0".split())            # unsupported kernel
    with pytest.raises(SystemExit):
        sweep.parse("128 128 128".split())                     # the driver wants all seven


def test_testbench_is_the_64_cube_sweep(sweep):
    cubes = sweep.shapes(sweep.parse("1 1 1 2 0 0 1".split()))
    assert len(cubes) == 64 and cubes[0] == (256, 256, 256) and cubes[-1] == (16384, 16384, 16384)
    assert all(m == k == n and m % 256 == 0 for m, k, n in cubes)
    assert sweep.shapes(sweep.parse("128 64 32 1 0 0 0".split())) == [(128, 64, 32)]
    assert len(sweep.shapes(sweep.parse("1 1 1 2 0 0 1 --max-dim 1024".split()))) == 4


def test_gflops_formula_and_dtype_pairs(sweep):
    # 100 calls of 1 ms each at 1024^3: 2 * 2^30 flop per ms = 2147.48 GFLOP/s
    assert sweep.gflops(1024, 1024, 1024, 100.0) == pytest.approx(2147.483648)
    assert sweep.PAIRS[1] == sweep.PAIRS[2] == (0, 0) and sweep.PAIRS[3] == (1, 1)
    assert sweep.PAIRS[5] == (0, 1) and sweep.PAIRS[7] == (1, 0)


def test_record_creates_the_directory_and_appends(sweep, tmp_path):
    d = str(tmp_path / "data")
    p = sweep.record_line(d, 2, 256, 256, 256, 1234.5)
    sweep.record_line(d, 2, 512, 512, 512, 99.0)
    assert os.path.basename(p) == "fp8_gemm_v2.csv"
    assert open(p).read().splitlines() == ["256,256,256,1234.5", "512,512,512,99.0"]
    assert os.path.basename(sweep.record_line(d, 9, 1, 1, 1, 1.0)) == "fp8_gemm_cublaslt.csv"


def test_jsonl_log_resumes_and_ignores_a_torn_last_line(sweep, tmp_path):
    log = str(tmp_path / "runs" / "sweep.jsonl")
    sweep.jsonl_append(log, {"m": 256, "k": 256, "n": 256, "kernel": 2, "gflops": 1.0})
    sweep.jsonl_append(log, {"m": 512, "k": 512, "n": 512, "kernel": 2, "gflops": 2.0})
    with open(log, "a") as f:
        f.write('{"m": 768, "k": 768, "n"')                  # a run killed in the middle of a line
    assert sweep.jsonl_done(log) == {(256, 256, 256, 2), (512, 512, 512, 2)}
    assert sweep.jsonl_done(str(tmp_path / "absent.jsonl")) == set()
    a = sweep.parse("1 1 1 2 0 1 1 --jsonl x.jsonl --resume --plot y.svg".split())
    assert a.jsonl == "x.jsonl" and a.resume and a.plot == "y.svg"


def test_plot_draws_one_line_per_csv(sweep, tmp_path):
    d = str(tmp_path / "data")
    assert sweep.plot_svg(d, str(tmp_path / "none.svg")) is None        # nothing recorded yet
    for size, ours, lt in ((256, 900.0, 1000.0), (512, 8000.0, 9000.0), (1024, 400000.0, 450000.0)):
        sweep.record_line(d, 2, size, size, size, ours)
        sweep.record_line(d, 9, size, size, size, lt)
    sweep.record_line(d, 2, 128, 64, 32, 5.0)                           # not a cube: left out of the plot
    series = sweep.read_csvs(d)
    assert set(series) == {"v2", "cublaslt"} and [m for m, _ in series["v2"]] == [256, 512, 1024]
    out = sweep.plot_svg(d, str(tmp_path / "plots" / "sweep.svg"))
    svg = open(out).read()
    assert svg.startswith("<svg") and svg.count("<polyline") == 2 and "cublaslt" in svg and "v2" in svg
