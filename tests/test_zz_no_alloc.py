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

import pytest
import torch

from __graft_entry__ import load_package

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
