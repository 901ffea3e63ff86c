// Host stand-ins that let the reference's UNMODIFIED benchmark driver
// (GEMM/gemm_main.cpp, compiled from where it lies) run on a machine without a
// GPU, so that its own CPU verification loop (gemm_main.cpp:45-52) and its own
// comparison (gemm_main.cpp:159-184) judge the oracle.  TEST INFRASTRUCTURE
// ONLY; never linked into the library.
//
//  - The CUDA runtime calls BmFN makes (gemm_main.cpp:59-64, :69-83, :161,
//    :185-187) become malloc / memcpy / free and no-op events.
//  - The eight gemm::GEMM / gemm::GEMM4 overloads (GEMM/include/gemm.cuh:12-55)
//    are answered by the oracle's restatement of the reference loop,
//    oracle_gemm_ref_float.  The driver then prints "MAx Error is 0.000000"
//    exactly when the restatement reproduces the reference's loop bit for bit
//    on the reference's own inputs.
//  - With ORACLE_DUMP_DIR set, the first call writes A, B and C there
//    (a.bin, b.bin, c.bin, meta.txt): those files become tests/golden fixtures.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

extern "C" void oracle_gemm_ref_float(int M, int K, int N, const uint8_t* A, int fmt_a,
                                      const uint8_t* B, int fmt_b, float* C, int threads);

extern "C" {
cudaError_t cudaMalloc(void** p, size_t n) { *p = std::malloc(n ? n : 1); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
cudaError_t cudaFree(void* p) { std::free(p); return cudaSuccess; }
cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) { std::memcpy(d, s, n); return cudaSuccess; }
cudaError_t cudaEventCreate(cudaEvent_t* e) { *e = nullptr; return cudaSuccess; }
cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t) { return cudaSuccess; }
cudaError_t cudaEventSynchronize(cudaEvent_t) { return cudaSuccess; }
cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t, cudaEvent_t) { *ms = 1.0f; return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t) { return "host stand-in"; }
}

namespace {
const void* g_last_a = nullptr;
const void* g_last_b = nullptr;
float* g_last_c = nullptr;
int g_last_m = -1, g_last_k = -1, g_last_n = -1;

void dump(const char* dir, int m, int k, int n, const uint8_t* a, int fa, const uint8_t* b, int fb, const float* c)
{
    auto put = [&](const char* name, const void* p, size_t bytes) {
        std::string path = std::string(dir) + "/" + name;
        FILE* f = std::fopen(path.c_str(), "wb");
        if (!f) { std::perror(path.c_str()); std::exit(2); }
        std::fwrite(p, 1, bytes, f);
        std::fclose(f);
    };
    put("a.bin", a, (size_t)m * k);
    put("b.bin", b, (size_t)n * k);
    put("c.bin", c, (size_t)m * n * sizeof(float));
    std::string path = std::string(dir) + "/meta.txt";
    FILE* f = std::fopen(path.c_str(), "w");
    std::fprintf(f, "%d %d %d %d %d\n", m, k, n, fa, fb);
    std::fclose(f);
}

cudaError_t answer(int m, int k, int n, const void* a, int fa, const void* b, int fb, float* c)
{
    // BmFN calls 120 times with identical arguments; compute once.
    if (a == g_last_a && b == g_last_b && c == g_last_c && m == g_last_m && k == g_last_k && n == g_last_n)
        return cudaSuccess;
    oracle_gemm_ref_float(m, k, n, (const uint8_t*)a, fa, (const uint8_t*)b, fb, c, 1);
    if (const char* dir = std::getenv("ORACLE_DUMP_DIR"))
        dump(dir, m, k, n, (const uint8_t*)a, fa, (const uint8_t*)b, fb, c);
    g_last_a = a; g_last_b = b; g_last_c = c; g_last_m = m; g_last_k = k; g_last_n = n;
    return cudaSuccess;
}
}  // namespace

namespace gemm {
typedef __nv_fp8_e5m2 e5m2;
typedef __nv_fp8_e4m3 e4m3;
cudaError_t GEMM(int m, int k, int n, const e4m3* __restrict__ a, const e4m3* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 0, b, 0, c); }
cudaError_t GEMM4(int m, int k, int n, const e4m3* __restrict__ a, const e4m3* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 0, b, 0, c); }
cudaError_t GEMM(int m, int k, int n, const e5m2* __restrict__ a, const e5m2* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 1, b, 1, c); }
cudaError_t GEMM4(int m, int k, int n, const e5m2* __restrict__ a, const e5m2* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 1, b, 1, c); }
cudaError_t GEMM(int m, int k, int n, const e4m3* __restrict__ a, const e5m2* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 0, b, 1, c); }
cudaError_t GEMM4(int m, int k, int n, const e4m3* __restrict__ a, const e5m2* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 0, b, 1, c); }
cudaError_t GEMM(int m, int k, int n, const e5m2* __restrict__ a, const e4m3* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 1, b, 0, c); }
cudaError_t GEMM4(int m, int k, int n, const e5m2* __restrict__ a, const e4m3* __restrict__ b, float* __restrict__ c) { return answer(m, k, n, a, 1, b, 0, c); }
}  // namespace gemm
