"""No-GPU checks of the boundary: the library loads, exports every declared symbol, and
rejects bad arguments before touching the device.  (No compute call is made here.)"""
import ctypes
import os
import re
import subprocess

import pytest

from __graft_entry__ import ROOT, load_package


@pytest.fixture(scope="module")
def pkg():
    p = load_package()
    if not os.path.exists(p._cabi.LIB_PATH):
        p._cabi.build()
    return p


def test_header_symbols_exported(pkg):
    header = open(os.path.join(ROOT, "include", "b200fp8.h")).read()
    diag = re.findall(r"#ifdef B200FP8_DIAGNOSTICS(.*?)#endif", header, flags=re.S)
    product = re.sub(r"#ifdef B200FP8_DIAGNOSTICS.*?#endif", "", header, flags=re.S)
    declared = set(re.findall(r"\b(b200fp8_[a-z0-9_]+)\s*\(", product))
    assert declared == set(pkg._cabi.DECLARED_SYMBOLS), declared ^ set(pkg._cabi.DECLARED_SYMBOLS)
    lib = pkg._cabi.lib()
    for sym in declared:
        assert getattr(lib, sym) is not None
    # what the header declares only for the diagnostics build is absent from the product library
    out = subprocess.run(["nm", "-D", "--defined-only", pkg._cabi.LIB_PATH], capture_output=True, text=True, check=True).stdout
    for sym in re.findall(r"\b(b200fp8_[a-z0-9_]+)\s*\(", "".join(diag)):
        assert sym not in out, sym


def test_reference_operator_symbols_exported(pkg):
    # the eight mangled names the reference's gemm_main.cpp imports (GEMM/include/gemm.cuh:12-55)
    out = subprocess.run(["nm", "-D", "--defined-only", pkg._cabi.LIB_PATH], capture_output=True, text=True, check=True).stdout
    for sym in pkg._cabi.OPERATOR_SYMBOLS:
        assert sym in out, sym
    assert len(pkg._cabi.OPERATOR_SYMBOLS) == 8


def test_version_string(pkg):
    assert b"sm_100a" in pkg._cabi.lib().b200fp8_version()


def test_invalid_arguments_return_invalid_value_without_launch(pkg):
    lib = pkg._cabi.lib()
    INVALID = 1  # cudaErrorInvalidValue
    fake = ctypes.c_void_p(0x1000)  # never dereferenced: validation happens first
    f = lib.b200fp8_gemm_rowcol_f32
    assert f(-1, 128, 128, fake, 0, fake, 0, fake, 2, None) == INVALID
    assert f(128, 128, 128, fake, 5, fake, 0, fake, 2, None) == INVALID       # bad dtype
    assert f(128, 128, 128, None, 0, fake, 0, fake, 2, None) == INVALID       # null A
    assert f(128, 128, 128, fake, 0, fake, 0, None, 2, None) == INVALID       # null C
    assert f(128, 72, 128, fake, 0, fake, 0, fake, 2, None) == INVALID        # K % 16 != 0
    assert f(128, 128, 128, ctypes.c_void_p(0x1008), 0, fake, 0, fake, 2, None) == INVALID  # misaligned A
    assert f(128, 128, 128, fake, 0, fake, 0, fake, 3, None) == INVALID       # depth must be 0, 2 or 4
    assert f(0, 128, 128, fake, 0, fake, 0, fake, 2, None) == 0               # empty problem: nothing to do
    assert f(128, 128, 0, fake, 0, fake, 0, fake, 2, None) == 0
    opt = pkg._cabi.Options(4, 0, 0, 0, 0)                                    # wrong struct size
    g = lib.b200fp8_gemm_rowcol_f32_ex
    assert g(128, 128, 128, fake, 0, 128, fake, 0, 128, fake, 128, ctypes.byref(opt), None) == INVALID
    opt = pkg._cabi.Options(ctypes.sizeof(pkg._cabi.Options), 0, 9, 0, 0)     # unknown kernel id
    assert g(128, 128, 128, fake, 0, 128, fake, 0, 128, fake, 128, ctypes.byref(opt), None) == INVALID
    opt = pkg._cabi.Options(ctypes.sizeof(pkg._cabi.Options), 0, 0, 0, 0)
    assert g(128, 128, 128, fake, 0, 64, fake, 0, 128, fake, 128, ctypes.byref(opt), None) == INVALID   # lda < k
    assert g(128, 128, 128, fake, 0, 128, fake, 0, 128, fake, 64, ctypes.byref(opt), None) == INVALID   # ldc < n
    assert lib.b200fp8_fill_normal(None, 16, 0, 1.0, 1, 0, None) == INVALID
    assert lib.b200fp8_fill_normal(fake, -1, 0, 1.0, 1, 0, None) == INVALID
    assert lib.b200fp8_device_status(None, 0) == INVALID


def test_host_mirror_rejects_cpu_tensors(pkg):
    import torch
    a = torch.zeros((16, 16), dtype=torch.float8_e4m3fn)
    out = torch.zeros((16, 16), dtype=torch.float32)
    with pytest.raises(ValueError):
        pkg.gemm.GEMM(16, 16, 16, a, a, out)
    with pytest.raises(TypeError):
        pkg.gemm.dtype_code(out)


def test_column_shards_partition_n(pkg):
    sh = pkg.shard
    for n in (32768, 8192, 1000, 257, 256, 1):
        for world in (1, 2, 3, 4, 8):
            parts = sh.all_shards(n, world)
            assert parts[0].n_begin == 0 and parts[-1].n_end == n
            for p, q in zip(parts, parts[1:]):
                assert p.n_end == q.n_begin
            assert sum(p.n for p in parts) == n
            assert all(p.n_begin % 256 == 0 or p.n_begin == n for p in parts)
    assert [p.n for p in sh.all_shards(32768, 8)] == [4096] * 8
    with pytest.raises(ValueError):
        sh.column_shard(10, 3, 2)


def test_python_wrappers_reject_bad_extents_before_the_call(pkg):
    """The C ABI sees only pointers, so the wrappers prove shapes, strides and extents first (no GPU needed: the
    checks come before the library call)."""
    import torch
    g = pkg.gemm
    t = torch.empty((4, 8))
    g._check_extent("t", t, 4, 8, 8)                                   # exact fit
    g._check_extent("view", torch.empty((4, 16))[:, :8], 4, 8, 16)     # a column block of a wider matrix (pitch 16)
    with pytest.raises(ValueError):
        g._check_extent("transposed", t.t(), 8, 4, 4)                  # rows are not contiguous
    with pytest.raises(ValueError):
        g._check_extent("short", t, 5, 8, 8)                           # one row more than the tensor holds
    with pytest.raises(ValueError):
        g._check_extent("pitch", t, 4, 8, 4)                           # pitch smaller than a row
    a = torch.empty((8, 32), dtype=torch.uint8).view(torch.float8_e4m3fn)
    b = torch.empty((16, 32), dtype=torch.uint8).view(torch.float8_e4m3fn)
    with pytest.raises(ValueError):
        g.gemm_ex(a, b, torch.empty((8, 16)))                          # host tensors: the operator takes device pointers
    with pytest.raises(ValueError):
        g.gemm_host(a, b, torch.empty((8, 15)))                        # out has the wrong shape
    with pytest.raises(ValueError):
        g.gemm_host(a, b, torch.empty((8, 16), dtype=torch.float64))   # out has the wrong dtype
    with pytest.raises(ValueError):
        g.gemm_host(a, b[:, :16], torch.empty((8, 16)))                # K mismatch
    with pytest.raises(ValueError):
        g.gemm_host(a, torch.empty((16, 64), dtype=torch.uint8).view(torch.float8_e4m3fn)[:, :32], torch.empty((8, 16)))  # not contiguous
