// Operator API of the B200 FP8 GEMM library, source-compatible with the reference's
// GEMM/include/gemm.cuh:6-55: the same typedefs and the same eight declarations, so code
// written against the reference header compiles and links against this library unchanged.
//
//   output[m][n] = sum_k a[m][k] * b[n][k]    a: row-major M x K, b: column-major K x N
//                                             (N rows of K), output: row-major M x N FP32
//
// Argument order is (m, k, n).  All pointers are device pointers; the call is asynchronous
// on the legacy default stream and returns the launch status.  GEMM uses a 2-deep
// shared-memory ring ("2-stage"), GEMM4 a 4-deep one ("4-stage").
#ifndef B200FP8_GEMM_CUH
#define B200FP8_GEMM_CUH
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

typedef __nv_fp8_e5m2 e5m2;
typedef __nv_fp8_e4m3 e4m3;

namespace gemm {

cudaError_t GEMM(int m, int k, int n, const e4m3* __restrict__ a_matrix, const e4m3* __restrict__ b_matrix,
                 float* __restrict__ output_matrix);
cudaError_t GEMM4(int m, int k, int n, const e4m3* __restrict__ a_matrix, const e4m3* __restrict__ b_matrix,
                  float* __restrict__ output_matrix);
cudaError_t GEMM(int m, int k, int n, const e5m2* __restrict__ a_matrix, const e5m2* __restrict__ b_matrix,
                 float* __restrict__ output_matrix);
cudaError_t GEMM4(int m, int k, int n, const e5m2* __restrict__ a_matrix, const e5m2* __restrict__ b_matrix,
                  float* __restrict__ output_matrix);
cudaError_t GEMM(int m, int k, int n, const e4m3* __restrict__ a_matrix, const e5m2* __restrict__ b_matrix,
                 float* __restrict__ output_matrix);
cudaError_t GEMM4(int m, int k, int n, const e4m3* __restrict__ a_matrix, const e5m2* __restrict__ b_matrix,
                  float* __restrict__ output_matrix);
cudaError_t GEMM(int m, int k, int n, const e5m2* __restrict__ a_matrix, const e4m3* __restrict__ b_matrix,
                 float* __restrict__ output_matrix);
cudaError_t GEMM4(int m, int k, int n, const e5m2* __restrict__ a_matrix, const e4m3* __restrict__ b_matrix,
                  float* __restrict__ output_matrix);

}  // namespace gemm
#endif
