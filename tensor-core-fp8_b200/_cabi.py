"""ctypes binding of include/b200fp8.h.

The shared library is built in-tree (csrc/Makefile).  There is no fallback: if the
library is missing, or a call reports a CUDA error, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

E4M3 = 0
E5M2 = 1

KERNEL_AUTO = 0
KERNEL_CTA1_N256 = 1
KERNEL_CTA1_N128 = 2
KERNEL_PAIR_N256 = 3
KERNEL_SKINNY = 4
KERNEL_PAIR_N512 = 5
KERNEL_PAIR_N128 = 6
KERNEL_CTA1_N64 = 7
KERNEL_SKINNY_STREAMK = 8

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
LIB_PATH = os.path.join(CSRC, "libb200fp8.so")
CMP_LIB_PATH = os.path.join(CSRC, "libb200fp8_cmp.so")

# every symbol include/b200fp8.h declares
DECLARED_SYMBOLS = (
    "b200fp8_gemm_rowcol_f32",
    "b200fp8_gemm_rowcol_f32_ex",
    "b200fp8_gemm_rowcol_scaled",
    "b200fp8_gemm_rowcol_epilogue",
    "b200fp8_gemv_f32",
    "b200fp8_spmm_bell_rowcol_f32",
    "b200fp8_spmv_bell_f32",
    "b200fp8_gemm_rowcol_f32_allgather",
    "b200fp8_gemm_rowcol_f32_host",
    "b200fp8_host_release",
    "b200fp8_gemm_rowcol_f32_noalloc",
    "b200fp8_multi_create",
    "b200fp8_multi_destroy",
    "b200fp8_multi_shard",
    "b200fp8_multi_upload",
    "b200fp8_multi_fill_normal",
    "b200fp8_multi_run",
    "b200fp8_multi_download",
    "b200fp8_fill_normal",
    "b200fp8_device_status",
    "b200fp8_enable_peer_access",
    "b200fp8_ipc_alloc",
    "b200fp8_ipc_open",
    "b200fp8_ipc_close",
    "b200fp8_ipc_free",
    "b200fp8_launch_count",
    "b200fp8_copy_2d_async",
    "b200fp8_l2_sides",
    "b200fp8_choose_kernel",
    "b200fp8_version",
)
# the reference's operator API (GEMM/include/gemm.cuh:12-55) as the C++ linker sees it
OPERATOR_SYMBOLS = tuple(
    f"_ZN4gemm{name}EiiiPK13__nv_fp8_{a}{b}Pf"
    for name in ("4GEMM", "5GEMM4")
    for a, b in (("e4m3", "S2_"), ("e5m2", "S2_"), ("e4m3", "PK13__nv_fp8_e5m2"), ("e5m2", "PK13__nv_fp8_e4m3"))
)


class Options(ctypes.Structure):
    _fields_ = [("struct_bytes", ctypes.c_int), ("depth", ctypes.c_int), ("kernel", ctypes.c_int),
                ("split_k", ctypes.c_int), ("max_ctas", ctypes.c_int)]


class EpilogueDesc(ctypes.Structure):
    """b200fp8_epilogue of include/b200fp8.h."""
    _fields_ = [("struct_bytes", ctypes.c_int), ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
                ("a_scale", ctypes.c_void_p), ("b_scale", ctypes.c_void_p), ("d_scale", ctypes.c_void_p),
                ("amax_d", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("bias_dtype", ctypes.c_int),
                ("activation", ctypes.c_int), ("a_row_scale", ctypes.c_void_p), ("b_row_scale", ctypes.c_void_p)]


class B200Fp8Error(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: CUDA error {code}")
        self.code = code


_lib = None


def build(verbose: bool = False) -> None:
    """Compile the CUDA library for sm_100a (nvcc cross-compiles without a GPU)."""
    subprocess.check_call(["make", "-C", CSRC, "all"] + ([] if verbose else ["-s"]))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        # B200FP8_LIBRARY selects another build of the same ABI (the diagnostics build, csrc/Makefile target `diag`)
        path = os.environ.get("B200FP8_LIBRARY") or LIB_PATH
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is not built; run `make -C {CSRC}` (there is no fallback path)")
        L = ctypes.CDLL(path)
        vp, ci, ll, ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong
        L.b200fp8_gemm_rowcol_f32.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci, vp]
        L.b200fp8_gemm_rowcol_f32_ex.argtypes = [ci, ci, ci, vp, ci, ll, vp, ci, ll, vp, ll,
                                                 ctypes.POINTER(Options), vp]
        L.b200fp8_gemm_rowcol_f32_allgather.argtypes = [ci, ci, ci, vp, ci, vp, ci, ctypes.POINTER(vp), vp, ci, ci, ll, ll,
                                                        ctypes.POINTER(Options), vp]
        L.b200fp8_gemm_rowcol_scaled.argtypes = [ci, ci, ci, vp, ci, ll, vp, ci, ll, vp, ci, ll, ctypes.c_float,
                                                 ctypes.c_float, vp, vp, ctypes.POINTER(Options), vp]
        L.b200fp8_gemm_rowcol_epilogue.argtypes = [ci, ci, ci, vp, ci, ll, vp, ci, ll, vp, ci, ll,
                                                   ctypes.POINTER(EpilogueDesc), ctypes.POINTER(Options), vp]
        L.b200fp8_gemv_f32.argtypes = [ci, ci, vp, ci, ll, vp, ci, vp, vp]
        L.b200fp8_spmm_bell_rowcol_f32.argtypes = [ci, ci, ci, vp, ci, ll, vp, ci, vp, ci, ll, vp, ll,
                                                   ctypes.POINTER(Options), vp]
        L.b200fp8_spmv_bell_f32.argtypes = [ci, ci, vp, ci, ll, vp, ci, vp, ci, vp, ctypes.POINTER(Options), vp]
        L.b200fp8_gemm_rowcol_f32_host.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci]
        L.b200fp8_gemm_rowcol_f32_noalloc.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, vp, vp]
        L.b200fp8_fill_normal.argtypes = [vp, ll, ci, ctypes.c_float, ull, ull, vp]
        L.b200fp8_multi_create.argtypes = [ci, ctypes.POINTER(ci), ci, ci, ci, ci, ci, ci, ctypes.POINTER(vp)]
        L.b200fp8_multi_destroy.argtypes = [vp]
        L.b200fp8_multi_shard.argtypes = [vp, ci, ctypes.POINTER(ci), ctypes.POINTER(ll), ctypes.POINTER(ll), ctypes.POINTER(vp),
                                          ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(ll)]
        L.b200fp8_multi_upload.argtypes = [vp, vp, vp]
        L.b200fp8_multi_fill_normal.argtypes = [vp, ctypes.c_float, ull, ctypes.c_float, ull]
        L.b200fp8_multi_run.argtypes = [vp, ci, ctypes.POINTER(Options), ctypes.POINTER(ctypes.c_float)]
        L.b200fp8_multi_download.argtypes = [vp, vp, ci]
        L.b200fp8_host_release.argtypes = []
        L.b200fp8_copy_2d_async.argtypes = [vp, ctypes.c_size_t, vp, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, vp]
        L.b200fp8_enable_peer_access.argtypes = [ci]
        L.b200fp8_ipc_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(vp), ctypes.c_char_p]
        L.b200fp8_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.b200fp8_ipc_close.argtypes = [vp]
        L.b200fp8_ipc_free.argtypes = [vp]
        L.b200fp8_device_status.argtypes = [ctypes.POINTER(ci), ci]
        L.b200fp8_launch_count.restype = ll
        L.b200fp8_l2_sides.argtypes = [ctypes.POINTER(ctypes.c_ulonglong)]
        L.b200fp8_l2_sides.restype = ctypes.c_int
        L.b200fp8_choose_kernel.argtypes = [ci, ci, ci]
        L.b200fp8_choose_kernel.restype = ci
        L.b200fp8_version.restype = ctypes.c_char_p
        _lib = L
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise B200Fp8Error(code, what)
