"""The sweep tool end to end on a GPU: one small shape per operator and the comparator, verified and recorded."""
import importlib.util
import os

import pytest

from __graft_entry__ import PKG_DIR, load_package

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sweep():
    spec = importlib.util.spec_from_file_location("tcfp8_sweep", os.path.join(PKG_DIR, "sweep.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("kernel", [1, 2, 5, 8])
def test_single_shape_verifies_and_records(sweep, tmp_path, kernel, capsys):
    d = str(tmp_path / "data")
    rc = sweep.main(f"384 512 640 {kernel} 1 1 0 --data-dir {d}".split(), pkg=load_package())
    assert rc == 0
    out = capsys.readouterr().out
    assert "verify:" in out and "pass" in out
    line = open(os.path.join(d, f"fp8_gemm_v{kernel}.csv")).read().strip().split(",")
    assert line[:3] == ["384", "512", "640"] and float(line[3]) > 0


def test_small_sweep_with_comparator(sweep, tmp_path):
    d = str(tmp_path / "data")
    rc = sweep.main(f"1 1 1 2 1 1 1 --max-dim 768 --cublaslt --data-dir {d}".split(), pkg=load_package())
    assert rc == 0
    ours = open(os.path.join(d, "fp8_gemm_v2.csv")).read().splitlines()
    lt = open(os.path.join(d, "fp8_gemm_cublaslt.csv")).read().splitlines()
    assert [l.split(",")[0] for l in ours] == ["256", "512", "768"] == [l.split(",")[0] for l in lt]
