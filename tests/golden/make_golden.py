"""Regenerates the fixtures in this directory from the REFERENCE's own code.

Needs the reference tree (--ref, default: the REF default of oracle/Makefile) and the CUDA toolkit
headers; it is run once where those exist and its outputs are committed, so the
tests themselves never touch the reference tree.

    python tests/golden/make_golden.py --ref <reference checkout>

What it records:

fp8_formats.npz
    decode_e4m3 / decode_e5m2 : float32 value of every byte 0..255, from the
        toolkit's host cast-to-float that the reference's CPU loop uses
        (GEMM/gemm_main.cpp:48).
    encode_in : float32 inputs = all 65536 bfloat16 bit patterns widened to
        float32, followed by hand-picked edge values (ties, subnormal
        boundaries, +-max, overflow, infinities, signed zeros).
    encode_e4m3 / encode_e5m2 : the byte the FP8 constructor from float gives
        for each input (round-to-nearest-even, saturate-to-finite), as called
        in GEMM/include/bm_test_utils.h:139.
    dense_e4m3 / dense_e5m2 : the first 32x128 matrix produced by the
        reference's MakeDenseMatrix (bm_test_utils.h:131-143) with a
        default-constructed engine, as BmFN calls it (gemm_main.cpp:32-36).

gemm_<name>.npz
    A, B, C of one run of the reference's unmodified gemm_main.cpp over host
    stand-ins (oracle/ref_cpu_stubs.cpp): A and B are the reference's own
    inputs, C is the oracle's restatement of the reference loop, and
    `ref_verdict` is the line the REFERENCE's comparison printed for that C
    against its own CPU loop ("MAx Error is 0.000000").  fmt_a / fmt_b:
    0 = e4m3, 1 = e5m2.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
ORACLE_DIR = os.path.join(ROOT, "oracle")

EDGE_VALUES = [
    0.0, -0.0, 1.0, -1.0, 448.0, -448.0, 449.0, 464.0, 463.99, 464.01, 480.0, 1000.0, -1000.0, 1e6, -1e6,
    57344.0, -57344.0, 61439.0, 61440.0, 61441.0, 65536.0, 1e9, float("inf"), float("-inf"),
    2.0 ** -6, 2.0 ** -7, 2.0 ** -9, 2.0 ** -10, 2.0 ** -10 * 1.0001, 2.0 ** -10 * 0.9999, 3 * 2.0 ** -10,
    2.0 ** -14, 2.0 ** -16, 2.0 ** -17, 2.0 ** -17 * 1.0001, 2.0 ** -17 * 0.9999, 3 * 2.0 ** -17,
    1.0625, 1.1875, 1.0624999, 1.0625001, 1.125, 1.375, 1.25, 0.3, -0.3, 0.1, 17.0, 18.0, 19.0, 20.0, 21.0, 22.0,
    240.0, 232.0, 248.0, 0.0146484375, 0.015625, 0.017578125,
]

# (name, M, K, N, reference kernel id): ids 2/3/5/7 pick the dtype pair in gemm_main.cpp:224-259
GEMM_CASES = [
    ("e4m3_e4m3_128", 128, 128, 128, 2),   # the reference's `make gemm_test` (GEMM/makefile:48-49)
    ("e5m2_e5m2_64x192x96", 64, 192, 96, 3),
    ("e4m3_e5m2_48x256x80", 48, 256, 80, 5),
    ("e5m2_e4m3_80x64x48", 80, 64, 48, 7),
    ("e4m3_e4m3_longk_32x2048x48", 32, 2048, 48, 1),
    ("e4m3_e4m3_ragged_33x80x17", 33, 80, 17, 1),
]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of the reference checkout (its GEMM/ directory is compiled in place)")
    args = ap.parse_args()

    subprocess.check_call(["make", "-s", "-C", ORACLE_DIR, "oracle", "ref", f"REF={args.ref}"])
    H = ctypes.CDLL(os.path.join(ORACLE_DIR, "_ref", "libref_harness.so"))
    H.ref_fp8_from_float.restype = ctypes.c_uint8
    H.ref_fp8_from_float.argtypes = [ctypes.c_float, ctypes.c_int]
    H.ref_fp8_to_float.restype = ctypes.c_float
    H.ref_fp8_to_float.argtypes = [ctypes.c_uint8, ctypes.c_int]
    H.ref_make_dense.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_uint8)]

    out = {}
    for fmt, name in ((0, "e4m3"), (1, "e5m2")):
        out[f"decode_{name}"] = np.array([H.ref_fp8_to_float(b, fmt) for b in range(256)], dtype=np.float32)
    bf16 = (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)
    enc_in = np.concatenate([bf16, np.array(EDGE_VALUES, dtype=np.float32)])
    out["encode_in"] = enc_in
    for fmt, name in ((0, "e4m3"), (1, "e5m2")):
        out[f"encode_{name}"] = np.array([H.ref_fp8_from_float(float(v), fmt) for v in enc_in], dtype=np.uint8)
        dense = np.empty((32, 128), dtype=np.uint8)
        H.ref_make_dense(32, 128, fmt, dense.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)))
        out[f"dense_{name}"] = dense
    np.savez_compressed(os.path.join(HERE, "fp8_formats.npz"), **out)

    exe = os.path.join(ORACLE_DIR, "_ref", "ref_gemm_cpu")
    for name, M, K, N, kernel in GEMM_CASES:
        with tempfile.TemporaryDirectory() as tmp:
            env = dict(os.environ, ORACLE_DUMP_DIR=tmp)
            text = subprocess.run([exe, str(M), str(K), str(N), str(kernel), "1", "0", "0"], env=env, cwd=tmp,
                                  check=True, capture_output=True, text=True).stdout
            verdict = [ln for ln in text.splitlines() if "MAx Error" in ln]
            assert len(verdict) == 1, text
            m, k, n, fa, fb = (int(v) for v in open(os.path.join(tmp, "meta.txt")).read().split())
            assert (m, k, n) == (M, K, N)
            A = np.fromfile(os.path.join(tmp, "a.bin"), dtype=np.uint8).reshape(M, K)
            B = np.fromfile(os.path.join(tmp, "b.bin"), dtype=np.uint8).reshape(N, K)
            C = np.fromfile(os.path.join(tmp, "c.bin"), dtype=np.float32).reshape(M, N)
        print(f"{name}: {verdict[0]}")
        np.savez_compressed(os.path.join(HERE, f"gemm_{name}.npz"), A=A, B=B, C=C, fmt_a=fa, fmt_b=fb,
                            ref_verdict=verdict[0], ref_kernel_id=kernel)
    return 0


if __name__ == "__main__":
    sys.exit(main())
