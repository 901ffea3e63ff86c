// Skinny (decode-shaped) FP8 GEMM for sm_100a: M <= 128 rows of A against a large B.
// The work is streaming B[N][K] once from HBM, so the kernel is organised around bytes
// in flight, not tensor-core occupancy:
//
//   * swap-AB: a CTA owns 128 rows of B (N rides the 128-lane UMMA M axis) and all of A's
//     rows padded to MP in {16,32,64,128} (the UMMA N axis; TMA zero-fills the padding),
//     so the accumulator is C^T: TMEM lane = n, column = m;
//   * split-K: grid = (N tiles) x (K splits); every CTA streams its K range through a deep
//     TMA ring; with more than one split the partial tiles go to scratch memory and the
//     LAST CTA to finish a tile (a counter per tile, no spinning) adds the partials in
//     split order -- the result does not depend on which CTA was last;
//   * two CTAs fit per SM, so one CTA's epilogue overlaps the other's stream.
//
// Same operator contract as the main kernel (reference: gemm::GEMM, GEMM/include/gemm.cuh:12-55;
// the reference's kernels write nothing at all for M < 128, GEMM/src/gemm.cu:45-47).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "gemm_sm100.cuh"

namespace b200fp8 {

constexpr int kSkinnyMaxM = 128;
constexpr int kSkinnyTileN = 128;
constexpr int kSkinnyThreads = 192;

struct SkinnyArgs {
    int M, N, K;
    int kb_total;        // ceil(K / 128)
    int kb_per_split;    // k-blocks per split (last split may be shorter, never empty)
    int splits;
    int stages;
    uint32_t idesc;
    float* C;
    long long ldc;
    float* partial;      // [splits][M][N] FP32, used when splits > 1
    unsigned int* counters;  // [n_tiles], zero between launches
    int* status;
};

template <int MP>
struct SkinnySmem {
    static constexpr int kBBytes = kSkinnyTileN * kBlockK;   // B rows: the UMMA "A" operand
    static constexpr int kABytes = MP * kBlockK;             // A rows: the UMMA "B" operand
    static constexpr int kStageBytes = kBBytes + kABytes;
    static constexpr int kMaxStages = 8;
    static constexpr int kTmemCols = MP < 32 ? 32 : MP;
    __host__ __device__ static constexpr int bar_off(int stages) { return stages * kStageBytes; }
    __host__ __device__ static constexpr int dynamic_bytes(int stages) { return stages * kStageBytes + 8 * (2 * kMaxStages + 1) + 32 + 1024; }
};

template <int MP>
__global__ void __launch_bounds__(kSkinnyThreads, 2)
gemm_fp8_skinny_kernel(const __grid_constant__ CUtensorMap tmap_b,   // B[N][K], box 128 rows
                       const __grid_constant__ CUtensorMap tmap_a,   // A[M][K], box MP rows
                       const SkinnyArgs args)
{
    using L = SkinnySmem<MP>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
    const int stages = args.stages;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const uint32_t bar_full = smem_base + L::bar_off(stages);
    const uint32_t bar_empty = bar_full + 8 * L::kMaxStages;
    const uint32_t bar_acc = bar_empty + 8 * L::kMaxStages;
    const int misc_off = L::bar_off(stages) + 8 * (2 * L::kMaxStages + 1);
    const uint32_t tmem_slot = smem_base + misc_off;
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + misc_off + 8);
    volatile unsigned int* last_flag = reinterpret_cast<volatile unsigned int*>(smem_gen + misc_off + 16);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        *last_flag = 0;
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        ptx::mbar_init(bar_acc, 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(tmem_slot, L::kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;

    const int n_tile = blockIdx.x;
    const int split = blockIdx.y;
    const int n0 = n_tile * kSkinnyTileN;
    const int kb0 = split * args.kb_per_split;
    const int kb1 = min(args.kb_total, kb0 + args.kb_per_split);

    if (warp == 0) {
        int s = 0;
        uint32_t ph = 0;
        int issued = 0;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
            if (!wait_bounded(bar_empty + 8 * s, ph ^ 1u, abort_flag, false)) {
                record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
                ok = false;
                break;
            }
            if (lane == 0) {
                const uint32_t b_dst = smem_base + s * L::kStageBytes;
                ptx::mbar_arrive_expect_tx(bar_full + 8 * s, L::kStageBytes);
                ptx::tma_load_2d(b_dst, &tmap_b, kb * kBlockK, n0, bar_full + 8 * s);
                ptx::tma_load_2d(b_dst + L::kBBytes, &tmap_a, kb * kBlockK, 0, bar_full + 8 * s);
            }
            __syncwarp();
            ++issued;
            if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (!ok) {
            const int pending = issued < stages ? issued : stages;
            for (int i = 0; i < pending; ++i) {
                if (s == 0) { s = stages; ph ^= 1u; }
                --s;
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(bar_full + 8 * s, ph) && ptx::globaltimer_ns() - t0 < kWaitLimitNs) {}
            }
        }
    } else if (warp == 1) {
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
            if (!wait_bounded(bar_full + 8 * s, ph, abort_flag, false)) {
                record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            if (lane == 0) {
                const uint32_t b_src = smem_base + s * L::kStageBytes;
                const uint64_t adesc = ptx::umma_desc_k128(b_src);                 // 128 rows of B
                const uint64_t bdesc = ptx::umma_desc_k128(b_src + L::kBBytes);    // MP rows of A
#pragma unroll
                for (int k = 0; k < kBlockK / 32; ++k)
                    ptx::umma_f8<1>(tmem_base, adesc + 2 * k, bdesc + 2 * k, args.idesc, (kb > kb0) || (k > 0));
                ptx::umma_commit(bar_empty + 8 * s);
            }
            __syncwarp();
            if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (ok && lane == 0) ptx::umma_commit(bar_acc);
        __syncwarp();
    } else {
        // ---------------- epilogue: 128 threads, thread = one column n of C ----------------
        const int q = warp & 3;
        const int n = n0 + q * 32 + lane;
        const bool n_ok = n < args.N;
        bool ok = wait_bounded(bar_acc, 0, abort_flag, false);
        if (!ok) record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
        __syncwarp();
        ptx::tc_fence_after();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        const bool direct = (args.splits == 1);
        float* out = direct ? args.C : args.partial + static_cast<long long>(split) * args.M * args.N;
        const long long ld = direct ? args.ldc : args.N;
        if (ok) {
#pragma unroll
            for (int c = 0; c < MP / 16; ++c) {
                uint32_t v[16];
                ptx::tmem_ld_32x16(t_addr + c * 16, v);
                ptx::tmem_ld_wait();
                if (n_ok) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c * 16 + j;
                        if (m < args.M) out[m * ld + n] = __uint_as_float(v[j]);   // a warp writes 128 contiguous bytes
                    }
                }
            }
        }
        if (!direct) {
            // publish this split's partial tile, then find out whether this CTA is the last of the tile
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 2 && lane == 0) {
                const unsigned int prev = atomicAdd(args.counters + n_tile, 1u);
                *last_flag = (prev == static_cast<unsigned int>(args.splits - 1)) ? 1u : 0u;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*last_flag) {
                __threadfence();
                if (n_ok) {
                    for (int m = 0; m < args.M; ++m) {
                        float acc = 0.0f;
                        const float* p = args.partial + static_cast<long long>(m) * args.N + n;
                        for (int s = 0; s < args.splits; ++s)
                            acc += __ldcg(p + static_cast<long long>(s) * args.M * args.N);
                        args.C[m * args.ldc + n] = acc;
                    }
                }
                if (warp == 2 && lane == 0) args.counters[n_tile] = 0;   // ready for the next launch
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem_base, L::kTmemCols);
    }
}

using SkinnyEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline cudaError_t skinny_encode(SkinnyEncodeFn enc, CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                                 uint64_t ld, uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld};
    const cuuint32_t box[2] = {kBlockK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Split count and ring depth chosen for bytes in flight: about two CTAs per SM.
inline void skinny_plan(int sm_count, int n, int k, int mp, int depth, int split_k, int* splits, int* kb_per_split,
                        int* stages) {
    const int n_tiles = (n + kSkinnyTileN - 1) / kSkinnyTileN;
    const int kb_total = (k + kBlockK - 1) / kBlockK;
    int s = split_k;
    if (s <= 0) {
        s = (2 * sm_count) / n_tiles;
        if (s < 1) s = 1;
        if (s > 16) s = 16;
    }
    if (s > kb_total) s = kb_total;
    int per = (kb_total + s - 1) / s;
    s = (kb_total + per - 1) / per;          // no empty split
    *splits = s;
    *kb_per_split = per;
    int st = depth;
    if (st <= 0) {
        const int stage_bytes = (kSkinnyTileN + mp) * kBlockK;
        st = (108 * 1024) / stage_bytes;     // two CTAs per SM
        if (st > 8) st = 8;
        if (st < 2) st = 2;
    }
    *stages = st;
}

// Scratch layout: a fixed 64 KiB block of per-tile counters (zero between launches), then the
// partial tiles [splits][M][N].  The fixed block keeps counters and partials apart whatever N is.
constexpr size_t kSkinnyCounterBytes = 64 * 1024;
constexpr int kSkinnyMaxTiles = static_cast<int>(kSkinnyCounterBytes / sizeof(unsigned int));

inline size_t skinny_scratch_bytes(int m, int n, int splits) {
    const size_t partial = splits > 1 ? static_cast<size_t>(splits) * m * n * sizeof(float) : 0;
    return kSkinnyCounterBytes + partial;
}

template <int MP>
cudaError_t launch_skinny_mp(const CUtensorMap& tb, const CUtensorMap& ta, const SkinnyArgs& args, int n_tiles,
                             cudaStream_t stream) {
    using L = SkinnySmem<MP>;
    auto kernel = gemm_fp8_skinny_kernel<MP>;
    static int attr_bytes[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int bytes = L::dynamic_bytes(args.stages);
    if (attr_bytes[dev] < bytes) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        attr_bytes[dev] = bytes;
    }
    kernel<<<dim3(n_tiles, args.splits, 1), kSkinnyThreads, bytes, stream>>>(tb, ta, args);
    return cudaGetLastError();
}

// Launches the skinny kernel with caller-provided scratch (counters first, partials after).
inline cudaError_t launch_skinny_with_scratch(int sm_count, int* status, void* scratch, SkinnyEncodeFn enc, int m, int k,
                                              int n, const void* a, long long lda, const void* b, long long ldb, float* c,
                                              long long ldc, int a_dtype, int b_dtype, int splits, int kb_per_split,
                                              int stages, cudaStream_t stream) {
    (void)sm_count;
    const int mp = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    const int n_tiles = (n + kSkinnyTileN - 1) / kSkinnyTileN;
    SkinnyArgs args{};
    args.M = m; args.N = n; args.K = k;
    args.kb_total = (k + kBlockK - 1) / kBlockK;
    args.kb_per_split = kb_per_split;
    args.splits = splits;
    args.stages = stages;
    args.idesc = make_idesc_f8(b_dtype, a_dtype, 128, mp);   // swapped: B feeds the UMMA A operand
    args.C = c; args.ldc = ldc;
    if (n_tiles > kSkinnyMaxTiles) return cudaErrorInvalidValue;
    args.counters = static_cast<unsigned int*>(scratch);
    args.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kSkinnyCounterBytes);
    args.status = status;
    CUtensorMap tb, ta;
    cudaError_t e;
    if ((e = skinny_encode(enc, &tb, b, k, n, ldb, kSkinnyTileN)) != cudaSuccess) return e;
    if ((e = skinny_encode(enc, &ta, a, k, m, lda, mp)) != cudaSuccess) return e;
    switch (mp) {
        case 16: return launch_skinny_mp<16>(tb, ta, args, n_tiles, stream);
        case 32: return launch_skinny_mp<32>(tb, ta, args, n_tiles, stream);
        case 64: return launch_skinny_mp<64>(tb, ta, args, n_tiles, stream);
        default: return launch_skinny_mp<128>(tb, ta, args, n_tiles, stream);
    }
}

// Library-owned scratch, grown on demand (counters must start at zero; the kernel re-zeroes them).
inline cudaError_t launch_skinny(int sm_count, int* status, void** scratch, size_t* scratch_bytes, SkinnyEncodeFn enc,
                                 int m, int k, int n, const void* a, long long lda, const void* b, long long ldb, float* c,
                                 long long ldc, int a_dtype, int b_dtype, int depth, int split_k, cudaStream_t stream) {
    const int mp = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    int splits, per, stages;
    skinny_plan(sm_count, n, k, mp, depth, split_k, &splits, &per, &stages);
    const size_t need = skinny_scratch_bytes(m, n, splits);
    if (*scratch_bytes < need) {
        if (*scratch) { cudaFree(*scratch); *scratch = nullptr; *scratch_bytes = 0; }   // cudaFree waits for running kernels
        cudaError_t e = cudaMalloc(scratch, need);
        if (e != cudaSuccess) return e;
        if ((e = cudaMemset(*scratch, 0, need)) != cudaSuccess) return e;
        *scratch_bytes = need;
    }
    return launch_skinny_with_scratch(sm_count, status, *scratch, enc, m, k, n, a, lda, b, ldb, c, ldc, a_dtype, b_dtype,
                                      splits, per, stages, stream);
}

}  // namespace b200fp8
