// cuBLASLt FP8 comparator for the benchmark: the same C = A * B^T (row-col layout, FP32
// output, no scaling) computed by the vendor library on the same buffers.  It is the
// performance bar the library is measured against, not part of the library: nothing in
// libb200fp8.so links or calls it.
//
// Like-for-like version of the reference's comparator (GEMM/src/cublas.cu:29-63, :72-103),
// which uses alpha = 2, beta = 1, scale pointers and no warm-up: here alpha = 1, beta = 0,
// no scale pointers, warm-up runs, and the fastest of the heuristic's candidates is kept.
//
// Column-major mapping: C_rowmajor[M][N] = D_colmajor[N][M] = op(A_lt) * op(B_lt) with
// A_lt = our B (col-major K x N, lda = K, transposed), B_lt = our A (col-major K x M, ldb = K).
#include <cublasLt.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <vector>

namespace {
cudaDataType_t fp8_type(int d) { return d == 0 ? CUDA_R_8F_E4M3 : CUDA_R_8F_E5M2; }

// the candidate chosen by the last b200fp8_cmp_cublaslt call, kept for b200fp8_cmp_cublaslt_run
struct Chosen {
    bool valid = false;
    int m = 0, k = 0, n = 0, a_dtype = 0, b_dtype = 0;
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    cublasLtMatmulAlgo_t algo;
};
Chosen g_chosen;
cublasLtHandle_t g_handle = nullptr;
void* g_workspace = nullptr;
const size_t kWorkspaceBytes = 64ull << 20;
}

extern "C" {

// Runs cuBLASLt on device buffers a [M][K], b [N][K] -> c [M][N] (FP32).  Tries up to
// `max_algos` heuristic candidates, `iters` timed back-to-back launches each after 3
// warm-ups, and leaves the fastest candidate's result in c.  Returns 0 on success,
// -1 when cuBLASLt offers no kernel for the dtype pair, or a positive cuBLAS/CUDA status.
// best_ms receives the mean milliseconds per launch of the fastest candidate.
int b200fp8_cmp_cublaslt(int m, int k, int n, const void* a, int a_dtype, const void* b, int b_dtype, float* c,
                         int iters, int max_algos, int fast_accum, float* best_ms, int* algos_found, void* stream_v)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const size_t ws_bytes = kWorkspaceBytes;
    if (!g_handle) {
        if (cublasLtCreate(&g_handle) != CUBLAS_STATUS_SUCCESS) return 1001;
        if (cudaMalloc(&g_workspace, ws_bytes) != cudaSuccess) return 1002;
    }
    cublasLtHandle_t handle = g_handle;
    void* workspace = g_workspace;
    if (g_chosen.valid) {
        cublasLtMatrixLayoutDestroy(g_chosen.la); cublasLtMatrixLayoutDestroy(g_chosen.lb);
        cublasLtMatrixLayoutDestroy(g_chosen.lc); cublasLtMatmulDescDestroy(g_chosen.op);
        g_chosen.valid = false;
    }
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    cublasLtMatmulPreference_t pref = nullptr;
    int rc = 0;
    const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
    const int8_t fa = static_cast<int8_t>(fast_accum ? 1 : 0);
    std::vector<cublasLtMatmulHeuristicResult_t> res(max_algos > 0 ? max_algos : 1);
    int found = 0;
    float best = -1.0f;
    int best_i = -1;
    const float alpha = 1.0f, beta = 0.0f;
    cudaEvent_t e0 = nullptr, e1 = nullptr;

#define LT(x) do { cublasStatus_t s_ = (x); if (s_ != CUBLAS_STATUS_SUCCESS) { rc = 2000 + static_cast<int>(s_); goto done; } } while (0)
    LT(cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F));
    LT(cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)));
    LT(cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)));
    LT(cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_FAST_ACCUM, &fa, sizeof(fa)));
    LT(cublasLtMatrixLayoutCreate(&la, fp8_type(b_dtype), k, n, k));
    LT(cublasLtMatrixLayoutCreate(&lb, fp8_type(a_dtype), k, m, k));
    LT(cublasLtMatrixLayoutCreate(&lc, CUDA_R_32F, n, m, n));
    LT(cublasLtMatmulPreferenceCreate(&pref));
    LT(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws_bytes, sizeof(ws_bytes)));
    {
        cublasStatus_t s = cublasLtMatmulAlgoGetHeuristic(handle, op, la, lb, lc, lc, pref, max_algos, res.data(), &found);
        if (s != CUBLAS_STATUS_SUCCESS || found == 0) { rc = -1; goto done; }
    }
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int i = 0; i < found; ++i) {
        bool ok = true;
        for (int w = 0; w < 3 && ok; ++w)
            ok = cublasLtMatmul(handle, op, &alpha, b, la, a, lb, &beta, c, lc, c, lc, &res[i].algo, workspace, ws_bytes,
                                stream) == CUBLAS_STATUS_SUCCESS;
        if (!ok) continue;
        cudaEventRecord(e0, stream);
        for (int it = 0; it < iters; ++it)
            cublasLtMatmul(handle, op, &alpha, b, la, a, lb, &beta, c, lc, c, lc, &res[i].algo, workspace, ws_bytes, stream);
        cudaEventRecord(e1, stream);
        if (cudaEventSynchronize(e1) != cudaSuccess) { rc = 1003; goto done; }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        ms /= iters;
        if (best < 0 || ms < best) { best = ms; best_i = i; }
    }
    if (best_i < 0) { rc = -1; goto done; }
    // leave the fastest candidate's output in c
    cublasLtMatmul(handle, op, &alpha, b, la, a, lb, &beta, c, lc, c, lc, &res[best_i].algo, workspace, ws_bytes, stream);
    if (cudaStreamSynchronize(stream) != cudaSuccess) rc = 1004;
    if (rc == 0) {
        g_chosen.valid = true;
        g_chosen.m = m; g_chosen.k = k; g_chosen.n = n; g_chosen.a_dtype = a_dtype; g_chosen.b_dtype = b_dtype;
        g_chosen.op = op; g_chosen.la = la; g_chosen.lb = lb; g_chosen.lc = lc; g_chosen.algo = res[best_i].algo;
        op = nullptr; la = lb = lc = nullptr;      // ownership moved
    }
done:
#undef LT
    if (best_ms) *best_ms = best;
    if (algos_found) *algos_found = found;
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (pref) cublasLtMatmulPreferenceDestroy(pref);
    if (la) cublasLtMatrixLayoutDestroy(la);
    if (lb) cublasLtMatrixLayoutDestroy(lb);
    if (lc) cublasLtMatrixLayoutDestroy(lc);
    if (op) cublasLtMatmulDescDestroy(op);
    return rc;
}

// Times `iters` back-to-back launches of the candidate chosen by the last b200fp8_cmp_cublaslt call
// (same shape and dtypes required; returns -2 otherwise).  No selection, no warm-up: for alternating
// comparisons under identical thermal conditions.
int b200fp8_cmp_cublaslt_run(int m, int k, int n, const void* a, int a_dtype, const void* b, int b_dtype, float* c,
                             int iters, float* mean_ms, void* stream_v)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const Chosen& ch = g_chosen;
    if (!ch.valid || ch.m != m || ch.k != k || ch.n != n || ch.a_dtype != a_dtype || ch.b_dtype != b_dtype) return -2;
    const float alpha = 1.0f, beta = 0.0f;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, stream);
    for (int it = 0; it < iters; ++it)
        cublasLtMatmul(g_handle, ch.op, &alpha, b, ch.la, a, ch.lb, &beta, c, ch.lc, c, ch.lc, &ch.algo, g_workspace,
                       kWorkspaceBytes, stream);
    cudaEventRecord(e1, stream);
    int rc = cudaEventSynchronize(e1) == cudaSuccess ? 0 : 1003;
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    if (mean_ms) *mean_ms = ms / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

// Enqueues ONE launch of the chosen candidate on `stream` and returns without synchronising, so that a
// caller can time batches over rotating buffers exactly as it times the library's own calls.
int b200fp8_cmp_cublaslt_enqueue(int m, int k, int n, const void* a, int a_dtype, const void* b, int b_dtype, float* c,
                                 void* stream_v)
{
    const Chosen& ch = g_chosen;
    if (!ch.valid || ch.m != m || ch.k != k || ch.n != n || ch.a_dtype != a_dtype || ch.b_dtype != b_dtype) return -2;
    const float alpha = 1.0f, beta = 0.0f;
    return cublasLtMatmul(g_handle, ch.op, &alpha, b, ch.la, a, ch.lb, &beta, c, ch.lc, c, ch.lc, &ch.algo, g_workspace,
                          kWorkspaceBytes, static_cast<cudaStream_t>(stream_v)) == CUBLAS_STATUS_SUCCESS ? 0 : 2001;
}

}  // extern "C"
