"""A broken pipeline must end the kernel, not hang the GPU.

Every wait inside the kernels is bounded.  This test makes one wait run out without any fault: with
B200FP8_DEBUG=512 the producer warp leaves the third k-block of its first tile unloaded, so the ring slot's
barrier is a flag that nothing sets.  The MMA warp's wait on it expires after about two seconds, the CTA
raises its abort flag, every role leaves its loop, TMEM is released and the kernel returns; the host then
reads a non-zero status word.  Afterwards the same context still runs a correct GEMM (K = 256 has no third
k-block, so nothing is skipped).  Runs in a child process because the switch is read once per process.
"""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

CHILD = r"""
import sys, time
sys.path.insert(0, %r)
import numpy as np, torch
from __graft_entry__ import load_package
from oracle import fp8_oracle as fo
g = load_package().gemm
torch.cuda.set_device(0)
for kernel in (2, 3):
    m, k, n = 512, 1024, 1024
    a = torch.empty((m, k), dtype=torch.float8_e4m3fn, device="cuda"); g.fill_normal(a, 1.0, 1)
    b = torch.empty((n, k), dtype=torch.float8_e4m3fn, device="cuda"); g.fill_normal(b, 1.0, 2)
    out = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    t0 = time.time()
    g.gemm_ex(a, b, out, kernel=kernel)
    torch.cuda.synchronize()                      # must return: no hang, no CUDA error
    dt = time.time() - t0
    st = g.device_status(reset=True)
    print("kernel", kernel, "status", st, "seconds", round(dt, 2))
    assert st in (101, 102, 103), st
    assert dt < 60
    # the context is intact: a problem without a third k-block computes correctly
    k2 = 256
    a2, b2 = a[:, :k2].contiguous(), b[:, :k2].contiguous()
    out2 = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    g.gemm_ex(a2, b2, out2, kernel=kernel)
    torch.cuda.synchronize()
    assert g.device_status() == 0
    C64, S = fo.gemm_f64(a2.view(torch.uint8).cpu().numpy(), 0, b2.view(torch.uint8).cpu().numpy(), 0)
    bad, worst, _ = fo.check_tolerance(out2.cpu().numpy(), C64, S)
    assert bad == 0, (bad, worst)
print("OK")
"""


def test_expired_wait_ends_kernel_with_status_and_context_survives():
    assert torch.cuda.is_available()
    env = dict(os.environ, B200FP8_DEBUG="512")
    res = subprocess.run([sys.executable, "-c", CHILD % ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "OK" in res.stdout
