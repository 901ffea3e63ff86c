// The reference's operator API (GEMM/include/gemm.cuh:12-55): eight overloads of
// gemm::GEMM / gemm::GEMM4, forwarded to the C ABI.  Linking the reference's unmodified
// benchmark driver (GEMM/gemm_main.cpp) against this object resolves exactly the symbols it
// imports.  GEMM is the "2-stage" entry (ring depth 2), GEMM4 the "4-stage" one (depth 4);
// both launch on the legacy default stream like the reference (GEMM/src/gemm.cu:273-276).
// B200FP8_OPERATOR_DEPTH in the environment (0 = as deep as fits, 2 or 4) overrides the depth of both names for
// callers that want the fastest kernel behind the reference's function names; results do not depend on the depth.
#include <cstdlib>
#include "../../include/gemm.cuh"
#include "../../include/b200fp8.h"

namespace gemm {

namespace {
int operator_depth(int by_name) {
    static const int forced = [] {
        const char* v = std::getenv("B200FP8_OPERATOR_DEPTH");
        if (!v) return -1;
        const int d = std::atoi(v);
        return (d == 0 || d == 2 || d == 4) ? d : -1;
    }();
    return forced >= 0 ? forced : by_name;
}
}  // namespace

#define B200FP8_FORWARD(NAME, ATYPE, AFMT, BTYPE, BFMT, DEPTH)                                            \
    cudaError_t NAME(int m, int k, int n, const ATYPE* __restrict__ a_matrix, const BTYPE* __restrict__ b_matrix, \
                     float* __restrict__ output_matrix) {                                                 \
        return static_cast<cudaError_t>(                                                                  \
            b200fp8_gemm_rowcol_f32(m, k, n, a_matrix, AFMT, b_matrix, BFMT, output_matrix, operator_depth(DEPTH), nullptr)); \
    }

B200FP8_FORWARD(GEMM, e4m3, B200FP8_E4M3, e4m3, B200FP8_E4M3, 2)
B200FP8_FORWARD(GEMM4, e4m3, B200FP8_E4M3, e4m3, B200FP8_E4M3, 4)
B200FP8_FORWARD(GEMM, e5m2, B200FP8_E5M2, e5m2, B200FP8_E5M2, 2)
B200FP8_FORWARD(GEMM4, e5m2, B200FP8_E5M2, e5m2, B200FP8_E5M2, 4)
B200FP8_FORWARD(GEMM, e4m3, B200FP8_E4M3, e5m2, B200FP8_E5M2, 2)
B200FP8_FORWARD(GEMM4, e4m3, B200FP8_E4M3, e5m2, B200FP8_E5M2, 4)
B200FP8_FORWARD(GEMM, e5m2, B200FP8_E5M2, e4m3, B200FP8_E4M3, 2)
B200FP8_FORWARD(GEMM4, e5m2, B200FP8_E5M2, e4m3, B200FP8_E4M3, 4)

#undef B200FP8_FORWARD

}  // namespace gemm
