"""The planner audit tool runs: AUTO and every forced kernel on a few small shapes, table written, exit code by threshold."""
import importlib.util
import json
import os

import pytest
import torch

from __graft_entry__ import load_package

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def load_tool():
    spec = importlib.util.spec_from_file_location("planner_audit", os.path.join(ROOT, "tensor-core-fp8_b200", "planner_audit.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_audit_times_auto_and_forced_kernels(tmp_path):
    assert torch.cuda.is_available()
    tool = load_tool()
    out = tmp_path / "audit.json"
    # a generous threshold: this checks the tool, not the planner (timings of 4 us kernels jitter)
    rc = tool.main(["512x512x512", "300x1024x3000", "64x2048x1024", "--threshold", "3.0", "--json", str(out)], pkg=load_package())
    assert rc == 0
    rows = json.loads(out.read_text())
    assert [(r["m"], r["k"], r["n"]) for r in rows] == [(512, 512, 512), (300, 1024, 3000), (64, 2048, 1024)]
    for r in rows:
        assert r["auto_us"] > 0 and r["best_us"] > 0 and r["chosen_over_best"] == pytest.approx(r["chosen_us"] / r["best_us"], rel=0.02)
        assert str(r["chosen_kernel"]) in r["us_by_kernel"]
        assert set(r["us_by_kernel"]) >= {"1", "2", "3", "6", "7"}
    assert set(rows[2]["us_by_kernel"]) >= {"4", "8"}          # M <= 128: the split-K kernels are timed too
    lib = load_package()._cabi.lib()
    assert lib.b200fp8_choose_kernel(16, 8192, 8192) == 4 and lib.b200fp8_choose_kernel(8192, 8192, 8192) == 3
    assert lib.b200fp8_choose_kernel(0, 64, 64) == -1
    # an impossible threshold flags every shape and turns the exit code
    assert tool.main(["512x512x512", "--threshold", "0.01"], pkg=load_package()) == 1
