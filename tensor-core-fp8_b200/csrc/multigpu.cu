// N-sharded GEMM over the GPUs of one box, driven from ONE process through the C ABI (include/b200fp8.h,
// b200fp8_multi_*).  The reference is single-GPU (its operator, GEMM/include/gemm.cuh:12-55, is what every shard
// calls); its caller is a C++ program (GEMM/gemm_main.cpp:28-194), so the multi-GPU plan is offered to such a
// caller without Python, process groups or IPC:
//
//   * device i of D owns rows [n_begin_i, n_end_i) of B (a contiguous slab of B's storage) and the same columns of
//     C; A is replicated.  The compute step exchanges nothing;
//   * one host thread per device inside the library: each sets its device, enqueues the operator on its own
//     stream and times it with events; the threads meet at a barrier before the first launch and the call reports
//     the MAXIMUM over the devices;
//   * with `gather` every device holds the full M x N matrix C and the kernels' epilogues store every finished
//     box into all of them (b200fp8_gemm_rowcol_f32_allgather) through peer mappings enabled with
//     cudaDeviceEnablePeerAccess -- plain stores only, no collective library, no TMA or library kernel on peer memory.
//
// The same device may be listed more than once (several shards on one GPU): the shards' kernels never wait for one
// another, so this is safe, and it lets the whole plan be exercised on a single GPU.
#include <cuda_runtime.h>
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/b200fp8.h"

struct b200fp8_multi {
    int world = 0;
    int m = 0, k = 0, n = 0;
    int a_dtype = 0, b_dtype = 0;
    int gather = 0;
    std::vector<int> device;
    std::vector<long long> n_begin, n_end;
    std::vector<void*> a, b;            // per shard: A (M x K), B slab (n_i x K)
    std::vector<float*> c;              // per shard: C block (M x n_i, pitch n_i) or, with gather, the full M x N
    std::vector<cudaStream_t> stream;
};

namespace {

// even split of N in units of 256 columns (the widest tile), remainder to the low shards
void column_shard(long long n, int rank, int world, long long* begin, long long* end) {
    const long long align = 256;
    const long long units = (n + align - 1) / align;
    const long long base = units / world, extra = units % world;
    const long long b = rank * base + std::min<long long>(rank, extra);
    const long long e = b + base + (rank < extra ? 1 : 0);
    *begin = std::min(n, b * align);
    *end = std::min(n, e * align);
}

// runs fn(i) on one host thread per shard and returns the first error
template <class F>
cudaError_t per_shard(int world, F fn) {
    std::vector<cudaError_t> rc(world, cudaSuccess);
    std::vector<std::thread> threads;
    threads.reserve(world);
    for (int i = 0; i < world; ++i) threads.emplace_back([&, i] { rc[i] = fn(i); });
    for (auto& t : threads) t.join();
    for (cudaError_t e : rc)
        if (e != cudaSuccess) return e;
    return cudaSuccess;
}

}  // namespace

extern "C" {

int b200fp8_multi_create(int num_shards, const int* devices, int m, int k, int n, int a_dtype, int b_dtype, int gather,
                         b200fp8_multi** out) {
    if (!out) return cudaErrorInvalidValue;
    *out = nullptr;
    if (num_shards < 1 || num_shards > 8 || !devices || m <= 0 || k <= 0 || n <= 0 || (k % 16)) return cudaErrorInvalidValue;
    if ((a_dtype != B200FP8_E4M3 && a_dtype != B200FP8_E5M2) || (b_dtype != B200FP8_E4M3 && b_dtype != B200FP8_E5M2))
        return cudaErrorInvalidValue;
    if (gather && (n % 4)) return cudaErrorInvalidValue;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return e;
    for (int i = 0; i < num_shards; ++i)
        if (devices[i] < 0 || devices[i] >= count) return cudaErrorInvalidDevice;
    b200fp8_multi* p = new b200fp8_multi;
    p->world = num_shards; p->m = m; p->k = k; p->n = n; p->a_dtype = a_dtype; p->b_dtype = b_dtype; p->gather = gather ? 1 : 0;
    p->device.assign(devices, devices + num_shards);
    p->n_begin.resize(num_shards); p->n_end.resize(num_shards);
    p->a.assign(num_shards, nullptr); p->b.assign(num_shards, nullptr); p->c.assign(num_shards, nullptr);
    p->stream.assign(num_shards, nullptr);
    for (int i = 0; i < num_shards; ++i) column_shard(n, i, num_shards, &p->n_begin[i], &p->n_end[i]);
    int prev = 0;
    cudaGetDevice(&prev);
    e = per_shard(num_shards, [&](int i) -> cudaError_t {
        cudaError_t r = cudaSetDevice(p->device[i]);
        if (r != cudaSuccess) return r;
        const long long ni = p->n_end[i] - p->n_begin[i];
        if ((r = cudaStreamCreateWithFlags(&p->stream[i], cudaStreamNonBlocking)) != cudaSuccess) return r;
        if ((r = cudaMalloc(&p->a[i], static_cast<size_t>(m) * k)) != cudaSuccess) return r;
        if ((r = cudaMalloc(&p->b[i], static_cast<size_t>(std::max<long long>(ni, 1)) * k)) != cudaSuccess) return r;
        const size_t c_elems = static_cast<size_t>(m) * (gather ? n : std::max<long long>(ni, 1));
        if ((r = cudaMalloc(reinterpret_cast<void**>(&p->c[i]), c_elems * sizeof(float))) != cudaSuccess) return r;
        if (gather)
            for (int j = 0; j < num_shards; ++j)
                if (p->device[j] != p->device[i] && (r = static_cast<cudaError_t>(b200fp8_enable_peer_access(p->device[j]))) != cudaSuccess)
                    return r;
        return cudaSuccess;
    });
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        b200fp8_multi_destroy(p);
        return e;
    }
    *out = p;
    return cudaSuccess;
}

int b200fp8_multi_destroy(b200fp8_multi* p) {
    if (!p) return cudaSuccess;
    int prev = 0;
    cudaGetDevice(&prev);
    for (int i = 0; i < p->world; ++i) {
        if (cudaSetDevice(p->device[i]) != cudaSuccess) continue;
        if (p->stream[i]) { cudaStreamSynchronize(p->stream[i]); cudaStreamDestroy(p->stream[i]); }
    }
    for (int i = 0; i < p->world; ++i) {       // every stream is idle by now: no kernel still stores into a peer's matrix
        if (cudaSetDevice(p->device[i]) != cudaSuccess) continue;
        if (p->a[i]) cudaFree(p->a[i]);
        if (p->b[i]) cudaFree(p->b[i]);
        if (p->c[i]) cudaFree(p->c[i]);
    }
    cudaSetDevice(prev);
    delete p;
    return cudaSuccess;
}

int b200fp8_multi_shard(const b200fp8_multi* p, int shard, int* device, long long* n_begin, long long* n_end, void** a,
                        void** b, float** c, long long* ldc) {
    if (!p || shard < 0 || shard >= p->world) return cudaErrorInvalidValue;
    if (device) *device = p->device[shard];
    if (n_begin) *n_begin = p->n_begin[shard];
    if (n_end) *n_end = p->n_end[shard];
    if (a) *a = p->a[shard];
    if (b) *b = p->b[shard];
    if (c) *c = p->c[shard];
    if (ldc) *ldc = p->gather ? p->n : (p->n_end[shard] - p->n_begin[shard]);
    return cudaSuccess;
}

int b200fp8_multi_upload(b200fp8_multi* p, const void* a_host, const void* b_host) {
    if (!p || !a_host || !b_host) return cudaErrorInvalidValue;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaError_t e = per_shard(p->world, [&](int i) -> cudaError_t {
        cudaError_t r = cudaSetDevice(p->device[i]);
        if (r != cudaSuccess) return r;
        const size_t ni = static_cast<size_t>(p->n_end[i] - p->n_begin[i]);
        if ((r = cudaMemcpyAsync(p->a[i], a_host, static_cast<size_t>(p->m) * p->k, cudaMemcpyHostToDevice, p->stream[i])) != cudaSuccess) return r;
        if (ni && (r = cudaMemcpyAsync(p->b[i], static_cast<const uint8_t*>(b_host) + static_cast<size_t>(p->n_begin[i]) * p->k,
                                       ni * p->k, cudaMemcpyHostToDevice, p->stream[i])) != cudaSuccess) return r;
        return cudaStreamSynchronize(p->stream[i]);
    });
    cudaSetDevice(prev);
    return e;
}

int b200fp8_multi_fill_normal(b200fp8_multi* p, float sigma_a, unsigned long long seed_a, float sigma_b, unsigned long long seed_b) {
    if (!p) return cudaErrorInvalidValue;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaError_t e = per_shard(p->world, [&](int i) -> cudaError_t {
        cudaError_t r = cudaSetDevice(p->device[i]);
        if (r != cudaSuccess) return r;
        const long long ni = p->n_end[i] - p->n_begin[i];
        if ((r = static_cast<cudaError_t>(b200fp8_fill_normal(p->a[i], static_cast<long long>(p->m) * p->k, p->a_dtype, sigma_a, seed_a, 0,
                                                              p->stream[i]))) != cudaSuccess) return r;
        // a shard regenerates exactly its slab of the full B from the element offset alone
        if (ni && (r = static_cast<cudaError_t>(b200fp8_fill_normal(p->b[i], ni * p->k, p->b_dtype, sigma_b, seed_b,
                                                                    static_cast<unsigned long long>(p->n_begin[i]) * p->k, p->stream[i]))) != cudaSuccess)
            return r;
        return cudaStreamSynchronize(p->stream[i]);
    });
    cudaSetDevice(prev);
    return e;
}

int b200fp8_multi_run(b200fp8_multi* p, int steps, const b200fp8_options* options, float* max_ms_per_step) {
    if (!p || steps < 1) return cudaErrorInvalidValue;
    if (options && options->struct_bytes != static_cast<int>(sizeof(b200fp8_options))) return cudaErrorInvalidValue;
    std::vector<float> ms(p->world, 0.0f);
    std::atomic<int> arrived{0};
    std::atomic<int> failed{0};
    int prev = 0;
    cudaGetDevice(&prev);
    cudaError_t e = per_shard(p->world, [&](int i) -> cudaError_t {
        cudaError_t r = cudaSetDevice(p->device[i]);
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        if (r == cudaSuccess) r = cudaEventCreate(&e0);
        if (r == cudaSuccess) r = cudaEventCreate(&e1);
        if (r == cudaSuccess) r = cudaStreamSynchronize(p->stream[i]);
        // host barrier: every shard's thread is ready (or has failed) before anyone launches; never waits on the GPU
        if (r != cudaSuccess) failed.store(1);
        arrived.fetch_add(1);
        while (arrived.load() < p->world) std::this_thread::yield();
        if (failed.load()) {
            if (e0) cudaEventDestroy(e0);
            if (e1) cudaEventDestroy(e1);
            return r != cudaSuccess ? r : cudaErrorUnknown;
        }
        const int ni = static_cast<int>(p->n_end[i] - p->n_begin[i]);
        cudaEventRecord(e0, p->stream[i]);
        for (int s = 0; s < steps && r == cudaSuccess && ni > 0; ++s) {
            if (p->gather)
                r = static_cast<cudaError_t>(b200fp8_gemm_rowcol_f32_allgather(p->m, p->k, ni, p->a[i], p->a_dtype, p->b[i], p->b_dtype,
                                                                               p->c.data(), nullptr, p->world, i, p->n, p->n_begin[i],
                                                                               options, p->stream[i]));
            else
                r = static_cast<cudaError_t>(b200fp8_gemm_rowcol_f32_ex(p->m, p->k, ni, p->a[i], p->a_dtype, p->k, p->b[i], p->b_dtype,
                                                                        p->k, p->c[i], ni, options, p->stream[i]));
        }
        cudaEventRecord(e1, p->stream[i]);
        const cudaError_t sync = cudaStreamSynchronize(p->stream[i]);
        if (r == cudaSuccess) r = sync;
        if (r == cudaSuccess) {
            float t = 0.0f;
            cudaEventElapsedTime(&t, e0, e1);
            ms[i] = t / steps;
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        return r;
    });
    cudaSetDevice(prev);
    if (e != cudaSuccess) return e;
    if (max_ms_per_step) *max_ms_per_step = *std::max_element(ms.begin(), ms.end());
    return cudaSuccess;
}

int b200fp8_multi_download(b200fp8_multi* p, float* c_host, int from_shard) {
    if (!p || !c_host) return cudaErrorInvalidValue;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaError_t e;
    if (p->gather) {
        // every shard holds the complete row-major matrix: one copy from the shard asked for
        if (from_shard < 0 || from_shard >= p->world) return cudaErrorInvalidValue;
        e = cudaSetDevice(p->device[from_shard]);
        if (e == cudaSuccess)
            e = cudaMemcpy(c_host, p->c[from_shard], static_cast<size_t>(p->m) * p->n * sizeof(float), cudaMemcpyDeviceToHost);
    } else {
        // column blocks: shard i's M x n_i block goes to columns [n_begin_i, n_end_i) of the row-major host matrix
        e = per_shard(p->world, [&](int i) -> cudaError_t {
            cudaError_t r = cudaSetDevice(p->device[i]);
            if (r != cudaSuccess) return r;
            const size_t ni = static_cast<size_t>(p->n_end[i] - p->n_begin[i]);
            if (!ni) return cudaSuccess;
            return cudaMemcpy2D(c_host + p->n_begin[i], static_cast<size_t>(p->n) * sizeof(float), p->c[i], ni * sizeof(float),
                                ni * sizeof(float), p->m, cudaMemcpyDeviceToHost);
        });
    }
    cudaSetDevice(prev);
    return e;
}

}  // extern "C"
