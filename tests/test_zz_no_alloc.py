"""The entry point that allocates nothing, against the regular one.

`b200fp8_gemm_rowcol_f32_noalloc` exists for callers that may not call cudaMalloc (a host program
that owns all device memory through its own pool, a process with a hard memory budget, a loop that
cannot afford an allocation's implicit synchronisation).  It keeps its scratch memory -- the
tile-pacing counter of the CTA-pair kernels -- in a static device array that every call shares and
that keeps the previous call's contents, so the test makes two calls in a row, the second one large
enough to use the counter again, and compares each with the regular entry point running the same
kernel: the results must be identical bit for bit (same kernel, same summation order), which is
stricter than the path's floating-point tolerance.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It passes alone in a fresh process as well as after the rest of the suite.
"""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

from __graft_entry__ import ROOT, load_package

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtypes", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn)])
def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row(dtypes):
    assert torch.cuda.is_available()
    pkg = load_package()
    g, lib = pkg.gemm, pkg._cabi.lib()
    torch.cuda.set_device(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # first call: a few tiles, ragged edges; second call: 1024 tile pairs, so the shared counter is used again
    for (m, k, n, kernel) in ((300, 272, 772, g.KERNEL_PAIR_N256), (8192, 256, 8192, g.KERNEL_PAIR_N256),
                              (8192, 256, 8192, g.KERNEL_PAIR_N256)):
        a = torch.empty((m, k), dtype=dtypes[0], device="cuda")
        b = torch.empty((n, k), dtype=dtypes[1], device="cuda")
        g.fill_normal(a, 1.0, 101 + m)
        g.fill_normal(b, 1.0, 202 + n)
        want = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        g.gemm_ex(a, b, want, kernel=kernel)
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        rc = lib.b200fp8_gemm_rowcol_f32_noalloc(m, k, n, a.data_ptr(), g.dtype_code(a), b.data_ptr(), g.dtype_code(b),
                                                 got.data_ptr(), status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got, want)
    # arguments are validated before anything touches the device
    assert lib.b200fp8_gemm_rowcol_f32_noalloc(128, 72, 128, a.data_ptr(), 0, b.data_ptr(), 0, got.data_ptr(), None, stream) == 1
    assert lib.b200fp8_gemm_rowcol_f32_noalloc(128, 128, 128, None, 0, b.data_ptr(), 0, got.data_ptr(), None, stream) == 1


def test_noalloc_wide_tile_branch_matches_the_wide_pair_kernel():
    """A problem of at least 16 rounds of 256 x 512 tiles with K >= 8192 takes the entry point's wide-tile kernel (with the
    pacing counter in the static array): bit for bit the regular entry point's kernel PAIR_N512."""
    pkg = load_package()
    g, lib = pkg.gemm, pkg._cabi.lib()
    torch.cuda.set_device(0)
    m, k, n = 8192, 8192, 28672
    a = torch.empty((m, k), dtype=torch.float8_e4m3fn, device="cuda")
    b = torch.empty((n, k), dtype=torch.float8_e4m3fn, device="cuda")
    g.fill_normal(a, 1.0, 7)
    g.fill_normal(b, 1.0, 8)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = torch.empty((m, n), dtype=torch.float32, device="cuda")
    g.gemm_ex(a, b, want, kernel=g.KERNEL_PAIR_N512)
    got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    rc = lib.b200fp8_gemm_rowcol_f32_noalloc(m, k, n, a.data_ptr(), 0, b.data_ptr(), 0, got.data_ptr(), status.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(got, want)


def test_noalloc_rejects_more_tiles_than_its_counter_is_specified_for():
    """m = n = 2^21 would be 2^25 wide tiles: beyond the stated maximum of 2^24.  The call must say so with
    cudaErrorInvalidValue before any descriptor is built or kernel launched; the pointers are never dereferenced."""
    pkg = load_package()
    g, lib = pkg.gemm, pkg._cabi.lib()
    torch.cuda.set_device(0)
    small = torch.empty(4096, dtype=torch.uint8, device="cuda")          # a valid, aligned device address; never accessed
    before = g.launch_count()
    rc = lib.b200fp8_gemm_rowcol_f32_noalloc(1 << 21, 8192, 1 << 21, small.data_ptr(), 0, small.data_ptr(), 0,
                                             small.data_ptr(), None, torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    assert g.launch_count() == before
    torch.cuda.synchronize()


_CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1])
import numpy as np
import torch
from __graft_entry__ import load_package
from oracle import fp8_oracle as fo
pkg = load_package()
lib = pkg._cabi.lib()
torch.cuda.set_device(0)
stream = torch.cuda.current_stream().cuda_stream
status = torch.zeros(1, dtype=torch.int32, device="cuda")
def operands(m, k, n, seed):
    rng = np.random.default_rng(seed)           # host-generated bytes: nothing but the entry point under test runs
    A = fo.fill_normal(m * k, 0, 1.0, seed).reshape(m, k)
    B = fo.fill_normal(n * k, 0, 1.0, seed + 1).reshape(n, k)
    return A, B, torch.from_numpy(A).cuda().view(torch.float8_e4m3fn), torch.from_numpy(B).cuda().view(torch.float8_e4m3fn)
# every buffer exists before the first call, so that torch's allocator is quiet afterwards
A1, B1, a1, b1 = operands(300, 272, 772, 3)
c1 = torch.full((300, 772), float("nan"), dtype=torch.float32, device="cuda")
A2, B2, a2, b2 = operands(8192, 128, 8192, 5)    # 1024 tile pairs: uses the pacing counter in the static array
c2 = torch.full((8192, 8192), float("nan"), dtype=torch.float32, device="cuda")
def call(m, k, n, a, b, c):
    rc = lib.b200fp8_gemm_rowcol_f32_noalloc(m, k, n, a.data_ptr(), 0, b.data_ptr(), 0, c.data_ptr(), status.data_ptr(), stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
call(300, 272, 772, a1, b1, c1)                  # first call on the device: set-up (module load, symbol address)
free0 = torch.cuda.mem_get_info()[0]
for _ in range(3):
    call(8192, 128, 8192, a2, b2, c2)
    call(300, 272, 772, a1, b1, c1)
free1 = torch.cuda.mem_get_info()[0]
assert free1 == free0, (free0, free1)            # the device's free memory did not move: nothing was allocated
assert int(status.item()) == 0
assert pkg.gemm.launch_count() == 7
C64, S = fo.gemm_f64(A1, 0, B1, 0)
bad, worst, _ = fo.check_tolerance(c1.cpu().numpy(), C64, S)
assert bad == 0, (bad, worst)
rows = np.arange(0, 8192, 257)
C64, S = fo.gemm_f64(np.ascontiguousarray(A2[rows]), 0, B2, 0)
bad, worst2, _ = fo.check_tolerance(c2[torch.from_numpy(rows).cuda()].cpu().numpy(), C64, S)
assert bad == 0, (bad, worst2)
print("NOALLOC_CHILD_OK", free0, worst, worst2)
"""


def test_noalloc_entry_alone_in_a_fresh_process_allocates_nothing():
    """A process that calls ONLY the entry point that allocates nothing (the regular entry points, which create the
    library's per-device buffers with cudaMalloc, never run in it): after the first call has loaded the kernels, the
    device's free memory (cudaMemGetInfo) is the same before and after a series of calls, one of which uses the pacing
    counter in the static array; results are checked against the FP64 oracle."""
    res = subprocess.run([sys.executable, "-c", _CHILD, ROOT], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "NOALLOC_CHILD_OK" in res.stdout
