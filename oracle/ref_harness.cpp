// Thin C wrapper around the REFERENCE's own host code, compiled from the
// reference sources where they lie (the include path is given by the Makefile;
// no reference source is copied here).  TEST INFRASTRUCTURE ONLY: used to pin
// the C restatement in fp8_oracle.c and to generate tests/golden/.
//
// Exposes:
//   - MakeDenseMatrix<T> of GEMM/include/bm_test_utils.h:131-143, called
//     exactly as BmFN calls it (a default-constructed engine passed by value,
//     GEMM/gemm_main.cpp:32-36);
//   - the toolkit FP8 conversions the reference relies on: the constructor
//     from float (bm_test_utils.h:139) and the cast to float
//     (gemm_main.cpp:48).
#include <cstdint>
#include <random>
#include <cuda_runtime_api.h>
#include "include/bm_test_utils.h"

extern "C" {

void ref_make_dense(int rows, int cols, int fmt, uint8_t* out)
{
    std::default_random_engine generator;
    if (fmt == 0)
        MakeDenseMatrix<__nv_fp8_e4m3>(rows, cols, reinterpret_cast<__nv_fp8_e4m3*>(out), generator);
    else
        MakeDenseMatrix<__nv_fp8_e5m2>(rows, cols, reinterpret_cast<__nv_fp8_e5m2*>(out), generator);
}

uint8_t ref_fp8_from_float(float x, int fmt)
{
    if (fmt == 0) { __nv_fp8_e4m3 v(x); return v.__x; }
    __nv_fp8_e5m2 v(x);
    return v.__x;
}

float ref_fp8_to_float(uint8_t byte, int fmt)
{
    if (fmt == 0) { __nv_fp8_e4m3 v; v.__x = byte; return (float)v; }
    __nv_fp8_e5m2 v;
    v.__x = byte;
    return (float)v;
}

}  // extern "C"
