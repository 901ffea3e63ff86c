// Seeded synthetic FP8 operands, generated on the device: element i of a tensor becomes
// fp8(sigma * z), z ~ N(0,1) from a counter-based generator keyed by (seed, i), converted with
// round-to-nearest-even and saturate-to-finite -- the conversion the reference's
// MakeDenseMatrix applies through the FP8 constructors (GEMM/include/bm_test_utils.h:131-143).
#pragma once
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace b200fp8 {

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111CBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float normal_sample(uint64_t seed, uint64_t idx) {
    const uint64_t h = splitmix64(seed ^ splitmix64(idx));
    const uint32_t u1 = static_cast<uint32_t>(h >> 40);
    const uint32_t u2 = static_cast<uint32_t>((h >> 16) & 0xFFFFFFu);
    const float f1 = (static_cast<float>(u1) + 1.0f) * (1.0f / 16777216.0f);
    const float f2 = static_cast<float>(u2) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(f1)) * cosf(6.28318530717958647692f * f2);
}

// one thread = 16 consecutive bytes (one 128-bit store when aligned)
__global__ void __launch_bounds__(256)
fill_normal_fp8_kernel(uint8_t* __restrict__ dst, long long count, int dtype, float sigma, uint64_t seed,
                       uint64_t index_offset)
{
    const long long chunks = (count + 15) / 16;
    const bool aligned = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    for (long long ch = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; ch < chunks;
         ch += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long base = ch * 16;
        uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float x = sigma * normal_sample(seed, index_offset + static_cast<uint64_t>(base + j));
            const __nv_fp8_storage_t b =
                __nv_cvt_float_to_fp8(x, __NV_SATFINITE, dtype == 0 ? __NV_E4M3 : __NV_E5M2);
            w[j >> 2] |= static_cast<uint32_t>(b) << (8 * (j & 3));
        }
        if (aligned && base + 16 <= count) {
            *reinterpret_cast<uint4*>(dst + base) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            for (int j = 0; j < 16 && base + j < count; ++j) dst[base + j] = static_cast<uint8_t>(w[j >> 2] >> (8 * (j & 3)));
        }
    }
}

inline cudaError_t launch_fill_normal(uint8_t* dst, long long count, int dtype, float sigma, uint64_t seed,
                                      uint64_t index_offset, int sm_count, cudaStream_t stream) {
    const long long chunks = (count + 15) / 16;
    long long blocks = (chunks + 255) / 256;
    const long long cap = static_cast<long long>(sm_count) * 8;     // a few resident blocks per SM, grid-stride beyond
    if (blocks > cap) blocks = cap;
    fill_normal_fp8_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(dst, count, dtype, sigma, seed, index_offset);
    return cudaGetLastError();
}

}  // namespace b200fp8
