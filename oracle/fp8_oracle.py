"""ctypes front-end for the CPU oracle (oracle/fp8_oracle.c).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg; the library itself never imports this module.

The C file restates the reference's CPU arithmetic for the FP8 GEMM path
(GEMM/gemm_main.cpp:45-52, GEMM/include/bm_test_utils.h:131-143 and the
toolkit FP8 formats the reference uses); see its header for the citations.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

E4M3 = 0
E5M2 = 1
REL_TOL = 1e-3
ABS_TOL = 1e-6

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int32)


def build(force: bool = False) -> str:
    """Compile liboracle.so (and, where the reference tree exists, oracle/_ref)."""
    src = os.path.join(_HERE, "fp8_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    return _LIB_PATH


def reference_root() -> str | None:
    """Root of the reference checkout: $REFERENCE_ROOT, else a directory `reference` beside this repository."""
    for cand in (os.environ.get("REFERENCE_ROOT"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "GEMM")):
            return cand
    return None


def build_ref(reference_root_dir: str | None = None) -> bool:
    """Build oracle/_ref from the reference sources where they lie; False if no reference checkout is found."""
    reference_root_dir = reference_root_dir or reference_root()
    if not reference_root_dir or not os.path.isdir(os.path.join(reference_root_dir, "GEMM")):
        return False
    subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={reference_root_dir}"])
    return True


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.oracle_fp8_decode.restype = ctypes.c_double
        L.oracle_fp8_decode.argtypes = [ctypes.c_uint8, ctypes.c_int]
        L.oracle_fp8_decode_table.argtypes = [ctypes.c_int, _f64p]
        L.oracle_fp8_encode.restype = ctypes.c_uint8
        L.oracle_fp8_encode.argtypes = [ctypes.c_float, ctypes.c_int]
        L.oracle_fp8_encode_array.argtypes = [_f32p, ctypes.c_int64, ctypes.c_int, _u8p]
        L.oracle_make_dense_uniform.argtypes = [ctypes.c_int64, ctypes.c_int, ctypes.c_uint32, _u8p]
        L.oracle_normal_sample.restype = ctypes.c_float
        L.oracle_normal_sample.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float]
        L.oracle_fill_normal_fp8.argtypes = [_u8p, ctypes.c_int64, ctypes.c_int, ctypes.c_float,
                                             ctypes.c_uint64, ctypes.c_uint64]
        L.oracle_gemm_ref_float.argtypes = [ctypes.c_int] * 3 + [_u8p, ctypes.c_int, _u8p, ctypes.c_int,
                                                                 _f32p, ctypes.c_int]
        L.oracle_gemm_ref_float_block.argtypes = ([ctypes.c_int] * 3 + [_u8p, ctypes.c_int, _u8p, ctypes.c_int,
                                                                        _f32p, ctypes.c_int64]
                                                  + [ctypes.c_int] * 5)
        L.oracle_gemm_f64_block.argtypes = [ctypes.c_int, _u8p, ctypes.c_int, _u8p, ctypes.c_int,
                                            _f64p, _f64p] + [ctypes.c_int] * 4
        L.oracle_gemm_f64_points.argtypes = [ctypes.c_int, _u8p, ctypes.c_int, _u8p, ctypes.c_int,
                                             _i32p, _i32p, ctypes.c_int64, _f64p, _f64p]
        L.oracle_check_tolerance.restype = ctypes.c_int64
        L.oracle_check_tolerance.argtypes = [_f32p, _f64p, _f64p, ctypes.c_int64, ctypes.c_double,
                                             ctypes.c_double, _f64p, ctypes.POINTER(ctypes.c_int64)]
        L.oracle_max_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def _u8(a: np.ndarray):
    assert a.dtype == np.uint8 and a.flags.c_contiguous
    return a.ctypes.data_as(_u8p)


def decode_table(fmt: int) -> np.ndarray:
    out = np.empty(256, dtype=np.float64)
    lib().oracle_fp8_decode_table(fmt, out.ctypes.data_as(_f64p))
    return out


def decode(bytes_: np.ndarray, fmt: int) -> np.ndarray:
    return decode_table(fmt)[np.asarray(bytes_, dtype=np.uint8)]


def encode(x: np.ndarray, fmt: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().oracle_fp8_encode_array(x.ctypes.data_as(_f32p), x.size, fmt, _u8(out))
    return out


def make_dense_uniform(rows: int, cols: int, fmt: int, state: int = 1) -> np.ndarray:
    """The reference's MakeDenseMatrix (bm_test_utils.h:131-143) restated."""
    out = np.empty((rows, cols), dtype=np.uint8)
    lib().oracle_make_dense_uniform(rows * cols, fmt, state, _u8(out))
    return out


def fill_normal(n: int, fmt: int, sigma: float, seed: int, index_offset: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.uint8)
    lib().oracle_fill_normal_fp8(_u8(out), n, fmt, sigma, seed, index_offset)
    return out


def gemm_ref_float(A: np.ndarray, fmt_a: int, B: np.ndarray, fmt_b: int, threads: int = 1,
                   rows=None, cols=None) -> np.ndarray:
    """The reference's CPU loop (gemm_main.cpp:45-52): A is [M][K], B is [N][K] bytes."""
    M, K = A.shape
    N, K2 = B.shape
    assert K == K2
    m0, m1 = rows if rows is not None else (0, M)
    n0, n1 = cols if cols is not None else (0, N)
    C = np.zeros((m1 - m0, n1 - n0), dtype=np.float32)
    if C.size and K >= 0:
        lib().oracle_gemm_ref_float_block(M, K, N, _u8(np.ascontiguousarray(A)), fmt_a,
                                          _u8(np.ascontiguousarray(B)), fmt_b,
                                          C.ctypes.data_as(_f32p), n1 - n0, m0, m1, n0, n1, threads)
    return C


def gemm_f64(A: np.ndarray, fmt_a: int, B: np.ndarray, fmt_b: int, rows=None, cols=None):
    """FP64 result and sum_k |a*b| for the block rows x cols (defaults: everything)."""
    M, K = A.shape
    N, _ = B.shape
    m0, m1 = rows if rows is not None else (0, M)
    n0, n1 = cols if cols is not None else (0, N)
    C = np.zeros((m1 - m0, n1 - n0), dtype=np.float64)
    S = np.zeros_like(C)
    if C.size:
        lib().oracle_gemm_f64_block(K, _u8(np.ascontiguousarray(A)), fmt_a, _u8(np.ascontiguousarray(B)), fmt_b,
                                    C.ctypes.data_as(_f64p), S.ctypes.data_as(_f64p), m0, m1, n0, n1)
    return C, S


def gemm_f64_points(A, fmt_a, B, fmt_b, ms, ns):
    ms = np.ascontiguousarray(ms, dtype=np.int32)
    ns = np.ascontiguousarray(ns, dtype=np.int32)
    C = np.zeros(ms.size, dtype=np.float64)
    S = np.zeros(ms.size, dtype=np.float64)
    lib().oracle_gemm_f64_points(A.shape[1], _u8(np.ascontiguousarray(A)), fmt_a,
                                 _u8(np.ascontiguousarray(B)), fmt_b,
                                 ms.ctypes.data_as(_i32p), ns.ctypes.data_as(_i32p), ms.size,
                                 C.ctypes.data_as(_f64p), S.ctypes.data_as(_f64p))
    return C, S


def check_tolerance(C: np.ndarray, C64: np.ndarray, S: np.ndarray, rel: float = REL_TOL, abs_tol: float = ABS_TOL):
    """Apply |C - C_ref| <= rel * sum_k|a*b| + abs_tol.  Returns (violations, worst ratio, worst index)."""
    C = np.ascontiguousarray(C, dtype=np.float32).ravel()
    C64 = np.ascontiguousarray(C64, dtype=np.float64).ravel()
    S = np.ascontiguousarray(S, dtype=np.float64).ravel()
    assert C.size == C64.size == S.size
    worst = ctypes.c_double(0.0)
    wi = ctypes.c_int64(-1)
    bad = lib().oracle_check_tolerance(C.ctypes.data_as(_f32p), C64.ctypes.data_as(_f64p),
                                       S.ctypes.data_as(_f64p), C.size, rel, abs_tol,
                                       ctypes.byref(worst), ctypes.byref(wi))
    return int(bad), float(worst.value), int(wi.value)


def max_threads() -> int:
    return int(lib().oracle_max_threads())


# ---------------------------------------------------------------- blocked-ELL sparse operands

BELL_BLOCK = 128


def make_bell_uniform(m: int, k: int, blocks: int, fmt: int, seed: int, sigma: float = 1.0):
    """A random blocked-ELL matrix with 128 x 128 blocks: (values [M][blocks*128] bytes, col_ind [ceil(M/128)][blocks]).

    Column indices follow the distribution of the reference's GenerateUniformBlockedELLIndex
    (GEMM/include/bm_test_utils.h:48-70): per block row a uniformly random subset of `blocks` of the
    ceil(K/128) block columns, in ascending order.  (The reference draws it with std::random_shuffle,
    whose random source is implementation-defined, so only the distribution can be restated.)"""
    rng = np.random.default_rng(seed)
    block_rows = (m + BELL_BLOCK - 1) // BELL_BLOCK
    block_cols = (k + BELL_BLOCK - 1) // BELL_BLOCK
    assert 0 <= blocks <= block_cols
    col_ind = np.empty((block_rows, blocks), dtype=np.int32)
    for r in range(block_rows):
        col_ind[r] = np.sort(rng.choice(block_cols, size=blocks, replace=False))
    values = fill_normal(m * blocks * BELL_BLOCK, fmt, sigma, seed + 1).reshape(m, blocks * BELL_BLOCK)
    return values, col_ind


def bell_to_dense(values: np.ndarray, col_ind: np.ndarray, k: int) -> np.ndarray:
    """Dense [M][K] bytes of a blocked-ELL matrix; blocks with an index < 0 or beyond K are dropped, columns of a
    block that reach past K are cut (what the kernels' zero-filled loads do).  Absent entries are +0 (byte 0)."""
    m = values.shape[0]
    dense = np.zeros((m, k), dtype=np.uint8)
    for r in range(col_ind.shape[0]):
        r0, r1 = r * BELL_BLOCK, min(m, (r + 1) * BELL_BLOCK)
        for j, c in enumerate(col_ind[r]):
            c0 = int(c) * BELL_BLOCK
            if c < 0 or c0 >= k:
                continue
            w = min(BELL_BLOCK, k - c0)
            assert not dense[r0:r1, c0:c0 + w].any(), "duplicate block column in a block row"
            dense[r0:r1, c0:c0 + w] = values[r0:r1, j * BELL_BLOCK:j * BELL_BLOCK + w]
    return dense
