// Skinny (decode-shaped) FP8 GEMM for sm_100a: M <= 128 rows of A against a large B.
// The work is streaming B[N][K] once from HBM, so the kernel is organised around bytes
// in flight, not tensor-core occupancy:
//
//   * swap-AB: a CTA owns 128 rows of B (N rides the 128-lane UMMA M axis) and all of A's
//     rows padded to MP in {16,32,64,128} (the UMMA N axis; TMA zero-fills the padding),
//     so the accumulator is C^T: TMEM lane = n, column = m;
//   * split-K inside a thread-block cluster: grid = (N tiles) x (K splits), the `splits`
//     CTAs of one N tile form a cluster (1 x splits x 1).  Every CTA streams its K range
//     through a deep TMA ring; the partial tiles are then parked in each CTA's own shared
//     memory and reduce-scattered through distributed shared memory: CTA r adds rows
//     r*rows_per.. of all partials in split order and writes them to C.  No scratch memory
//     in HBM, no atomics, and the result does not depend on timing;
//   * two CTAs fit per SM, so one CTA's epilogue overlaps the other's stream.
//
// Same operator contract as the main kernel (reference: gemm::GEMM, GEMM/include/gemm.cuh:12-55;
// the reference's kernels write nothing at all for M < 128, GEMM/src/gemm.cu:45-47).
#pragma once
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "gemm_sm100.cuh"

namespace b200fp8 {

constexpr int kSkinnyMaxM = 128;
constexpr int kSkinnyTileN = 128;
constexpr int kSkinnyThreads = 192;       // producer warp, MMA warp, four epilogue warps
// For M > 32 the reduce-scatter moves 16-64 KiB per CTA through distributed shared memory, and a warp's remote loads
// do not overlap each other (about half a microsecond per round): the CTA is launched with extra warps that do
// nothing but help with that phase.
constexpr int kSkinnyThreadsWide = 512;
constexpr int kSkinnyMaxSplits = 8;      // portable cluster size

struct SkinnyArgs {
    int M, N, K;
    int kb_total;        // ceil(K / 128)
    int kb_per_split;    // k-blocks per split (last split may be shorter, never empty)
    int splits;          // = cluster size along y
    int stages;
    int vec_store;       // 1: C rows are 16-byte aligned (ldc % 4 == 0 and C % 16 == 0)
    uint32_t idesc;
    float* C;
    long long ldc;
    int* status;
    // Blocked-ELL form of the LARGE operand B (128 x 128 blocks): tmap_b describes the compact values matrix
    // [N][kb_total * 128], and k-block kb of N-tile nt multiplies the columns [col * 128, col * 128 + 128) of A with
    // col = ell_col_ind[nt * kb_total + kb]; col < 0 or beyond K is a padding block (zeros are loaded for both).
    const int* ell_col_ind;
    int ell_oob_a, ell_oob_b;   // 128-aligned k coordinates beyond A's K / beyond the compact B
    long long* trace;    // diagnostics: eight globaltimer stamps per CTA (nullptr = off)
    int pdl;             // host only: launch with programmatic stream serialization
    int l2_prefetch;     // k-blocks of this CTA's first rows of B requested into L2 before the grid dependency wait
    Epilogue epi;        // extended epilogue (alpha, beta, scales, 16-bit output); inactive for the plain operator
};

// one element of D (column n) under the extended epilogue; `amax` is the thread's running |t| maximum
template <class Args>
__device__ __forceinline__ void skinny_store_epi(const Args& args, float alpha, float dscale, long long idx, int m, int n,
                                                 float acc, float& amax) {
    if (args.epi.b_row_scale != nullptr) acc *= __ldg(args.epi.b_row_scale + n);
    if (args.epi.a_row_scale != nullptr) alpha *= __ldg(args.epi.a_row_scale + m);
    float v = alpha * acc;
    if (args.epi.beta != 0.0f) v += args.epi.beta * load_out(args.C, idx, args.epi.out_dtype);
    if (args.epi.bias != nullptr) v += load_out(args.epi.bias, n, args.epi.bias_dtype);
    v = activate(v, args.epi.activation);
    amax = fmaxf(amax, fabsf(v));
    store_out(args.C, idx, dscale * v, args.epi.out_dtype);
}

template <int MP>
struct SkinnySmem {
    static constexpr int kBBytes = kSkinnyTileN * kBlockK;   // B rows: the UMMA "A" operand
    static constexpr int kABytes = MP * kBlockK;             // A rows: the UMMA "B" operand
    static constexpr int kStageBytes = kBBytes + kABytes;
    static constexpr int kMaxStages = 8;
    static constexpr int kTmemCols = MP < 32 ? 32 : MP;
    static constexpr int kPartialBytes = MP * kSkinnyTileN * 4;   // parked partial tile [m][n]; fits in two ring slots
    __host__ __device__ static constexpr int bar_off(int stages) { return stages * kStageBytes; }
    __host__ __device__ static constexpr int dynamic_bytes(int stages) { return stages * kStageBytes + 8 * (2 * kMaxStages + 1) + 32 + 1024; }
};

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr) : "memory");
    return v;
}

__device__ __forceinline__ float4 ld_local_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

template <int MP, int THREADS>
__global__ void __launch_bounds__(THREADS, THREADS <= kSkinnyThreads ? 2 : 1)
gemm_fp8_skinny_kernel(const __grid_constant__ CUtensorMap tmap_b,   // B[N][K], box 128 rows
                       const __grid_constant__ CUtensorMap tmap_a,   // A[M][K], box MP rows
                       const SkinnyArgs args)
{
    using L = SkinnySmem<MP>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
    const int stages = args.stages;
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // provably warp-uniform
    const int lane = threadIdx.x & 31;
    const bool clustered = args.splits > 1;

    const uint32_t bar_full = smem_base + L::bar_off(stages);
    const uint32_t bar_empty = bar_full + 8 * L::kMaxStages;
    const uint32_t bar_acc = bar_empty + 8 * L::kMaxStages;
    const int misc_off = L::bar_off(stages) + 8 * (2 * L::kMaxStages + 1);
    const uint32_t tmem_slot = smem_base + misc_off;
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + misc_off + 8);

    long long* trace = (kDiagnostics && args.trace) ? args.trace + 8ll * (blockIdx.y * gridDim.x + blockIdx.x) : nullptr;   // diagnostics build only
    if (trace && threadIdx.x == 0) trace[0] = static_cast<long long>(ptx::globaltimer_ns());
    if (threadIdx.x == 0) {
        *abort_flag = 0;
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
    if (warp == 0 && args.l2_prefetch > 0 && args.ell_col_ind == nullptr) {
        // The first blocks of B this CTA will stream, requested into L2 before the wait below.  A prefetch changes no
        // data anywhere (L2 is the point of coherence: a line the previous kernel still writes stays correct); it only
        // starts the first HBM round trip while the previous kernel of the stream drains.
        if (ptx::elect_one()) {
            const int first = blockIdx.y * args.kb_per_split;
            const int last = min(args.kb_total, first + min(args.kb_per_split, args.l2_prefetch));
            for (int kb = first; kb < last; ++kb) {
                asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
                             ::"l"(reinterpret_cast<uint64_t>(&tmap_b)), "r"(kb * kBlockK), "r"(static_cast<int>(blockIdx.x) * kSkinnyTileN) : "memory");
                // A is the same for every N tile: a few CTAs request it for all (it was evicted if B is larger than L2)
                if (blockIdx.x < 2)
                    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
                                 ::"l"(reinterpret_cast<uint64_t>(&tmap_a)), "r"(kb * kBlockK), "r"(0) : "memory");
            }
        }
        __syncwarp();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;
    // Everything above touched only this CTA's own resources (and hinted L2) and may overlap the previous kernel's
    // tail; global memory (operands, C, the status word) is touched only after the grids before this one are complete.
    ptx::griddep_wait();
    ptx::griddep_launch_dependents();
    if (trace && threadIdx.x == 0) trace[1] = static_cast<long long>(ptx::globaltimer_ns());

    float epi_alpha = 1.0f, epi_dscale = 1.0f, epi_amax = 0.0f;
    if (args.epi.active) {
        epi_alpha = args.epi.alpha;
        if (args.epi.a_scale) epi_alpha *= *args.epi.a_scale;
        if (args.epi.b_scale) epi_alpha *= *args.epi.b_scale;
        if (args.epi.d_scale) epi_dscale = *args.epi.d_scale;
    }
    const int n_tile = blockIdx.x;
    const int split = blockIdx.y;                  // = rank in the cluster (1 x splits x 1)
    const int n0 = n_tile * kSkinnyTileN;
    const int kb0 = split * args.kb_per_split;
    const int kb1 = min(args.kb_total, kb0 + args.kb_per_split);

    if (warp == 0) {
        int s = 0;
        uint32_t ph = 0;
        int issued = 0;
        bool ok = true;
        // blocked-ELL B: lane l holds the column block of k-block (chunk base + l); the next 32 are prefetched
        const int* ell_row = nullptr;
        int ell_cur = -1, ell_nxt = -1;
        if (args.ell_col_ind != nullptr) {
            ell_row = args.ell_col_ind + static_cast<long long>(n_tile) * args.kb_total;
            if (kb0 + lane < kb1) ell_nxt = ell_row[kb0 + lane];
        }
        for (int kb = kb0; kb < kb1; ++kb) {
            if (!wait_bounded(bar_empty + 8 * s, ph ^ 1u, abort_flag, false)) {
                record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
                ok = false;
                break;
            }
            int ka = kb * kBlockK, kbx = kb * kBlockK;               // k coordinates of the A and B boxes
            if (ell_row != nullptr) {
                const int rel = kb - kb0;
                if ((rel & 31) == 0) {
                    ell_cur = ell_nxt;
                    ell_nxt = (kb + 32 + lane < kb1) ? ell_row[kb + 32 + lane] : -1;
                }
                const int col = __shfl_sync(0xffffffffu, ell_cur, rel & 31);
                if (col < 0 || col >= args.ell_oob_a / kBlockK) { ka = args.ell_oob_a; kbx = args.ell_oob_b; }
                else ka = col * kBlockK;
            }
            const uint32_t b_dst = smem_base + s * L::kStageBytes;
            if (ptx::elect_one()) {
                ptx::mbar_arrive_expect_tx(bar_full + 8 * s, L::kStageBytes);
                ptx::tma_load_2d(b_dst, &tmap_b, kbx, n0, bar_full + 8 * s);
                ptx::tma_load_2d(b_dst + L::kBBytes, &tmap_a, ka, 0, bar_full + 8 * s);
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
            if (trace && kb == kb0 && lane == 0) trace[2] = static_cast<long long>(ptx::globaltimer_ns());
            const uint32_t b_src = smem_base + s * L::kStageBytes;
            const uint64_t adesc = ptx::umma_desc_k128(b_src);                 // 128 rows of B
            const uint64_t bdesc = ptx::umma_desc_k128(b_src + L::kBBytes);    // MP rows of A
            if (ptx::elect_one()) {
#pragma unroll
                for (int k = 0; k < kBlockK / 32; ++k)
                    ptx::umma_f8<1>(tmem_base, adesc + 2 * k, bdesc + 2 * k, args.idesc, (kb > kb0) || (k > 0));
                ptx::umma_commit(bar_empty + 8 * s);
            }
            __syncwarp();
            if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (ok && ptx::elect_one()) ptx::umma_commit(bar_acc);
        __syncwarp();
        if (trace && lane == 0) trace[3] = static_cast<long long>(ptx::globaltimer_ns());
    } else if (warp < kSkinnyThreads / 32) {
        // ---------------- epilogue: 128 threads, thread = one column n of C ----------------
        // bar_acc completes after every MMA of this CTA has finished, i.e. after the ring's
        // shared memory was last read and long after it was last written: it is free to reuse.
        const int q = warp & 3;
        const int n_local = q * 32 + lane;
        bool ok = wait_bounded(bar_acc, 0, abort_flag, false);
        if (!ok) record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
        if (trace && warp == 2 && lane == 0) trace[4] = static_cast<long long>(ptx::globaltimer_ns());
        __syncwarp();
        ptx::tc_fence_after();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        if (ok) {
            float* park = reinterpret_cast<float*>(smem_gen);      // [m][128] partial tile
#pragma unroll
            for (int c = 0; c < MP / 16; ++c) {
                if (c * 16 < args.M) {
                    uint32_t v[16];
                    ptx::tmem_ld_32x16(t_addr + c * 16, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c * 16 + j;
                        // parked even without K-splits: row-wise 16-byte stores from shared memory by all threads are
                        // several times faster than 4-byte stores straight from the TMEM read-out (28 -> 7 us at M = 128)
                        if (m < args.M) park[m * kSkinnyTileN + n_local] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }

    {
        // ---------------- reduce-scatter across the cluster through distributed shared memory ----------------
        // (a single split owns all rows and only reads its own parked tile)
        if (clustered) { ptx::cluster_arrive(); ptx::cluster_wait(); }
        else __syncthreads();
        if (trace && threadIdx.x == 0) trace[5] = static_cast<long long>(ptx::globaltimer_ns());
        const int rows_per = (args.M + args.splits - 1) / args.splits;
        const int m_begin = split * rows_per;
        const int m_end = min(args.M, m_begin + rows_per);
        const int items = max(0, m_end - m_begin) * (kSkinnyTileN / 4);      // float4 groups
        if (*abort_flag == 0) {
            for (int i = threadIdx.x; i < items; i += THREADS) {
                const int m = m_begin + i / (kSkinnyTileN / 4);
                const int cg = i % (kSkinnyTileN / 4);
                const uint32_t local = smem_base + static_cast<uint32_t>((m * kSkinnyTileN + cg * 4) * 4);
                float4 part[kSkinnyMaxSplits];
#pragma unroll
                for (int s = 0; s < kSkinnyMaxSplits; ++s)
                    if (s < args.splits) part[s] = (s == split) ? ld_local_f4(local) : ld_cluster_f4(ptx::mapa(local, s));
                float4 acc = part[0];
#pragma unroll
                for (int s = 1; s < kSkinnyMaxSplits; ++s)
                    if (s < args.splits) { acc.x += part[s].x; acc.y += part[s].y; acc.z += part[s].z; acc.w += part[s].w; }
                const int n = n0 + cg * 4;
                float* dst = args.C + m * args.ldc + n;
                if (args.epi.active) {
                    const long long idx = m * args.ldc + n;
                    if (n < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx, static_cast<int>(m), n, acc.x, epi_amax);
                    if (n + 1 < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx + 1, static_cast<int>(m), n + 1, acc.y, epi_amax);
                    if (n + 2 < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx + 2, static_cast<int>(m), n + 2, acc.z, epi_amax);
                    if (n + 3 < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx + 3, static_cast<int>(m), n + 3, acc.w, epi_amax);
                } else if (args.vec_store && n + 3 < args.N) {
                    *reinterpret_cast<float4*>(dst) = acc;
                } else {
                    if (n < args.N) dst[0] = acc.x;
                    if (n + 1 < args.N) dst[1] = acc.y;
                    if (n + 2 < args.N) dst[2] = acc.z;
                    if (n + 3 < args.N) dst[3] = acc.w;
                }
            }
        }
        if (trace && threadIdx.x == 0) trace[6] = static_cast<long long>(ptx::globaltimer_ns());
        // Peers may still be reading this CTA's shared memory: it must not exit before all of them have arrived
        // here too.  The wait for that comes last, so that the rest of the teardown overlaps the barrier's latency.
        __syncwarp();
        if (clustered) ptx::cluster_arrive();
    }
    __syncwarp();
    if (args.epi.amax != nullptr) amax_merge_warp(args.epi.amax, epi_amax);

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem_base, L::kTmemCols);
    }
    __syncwarp();
    if (clustered) ptx::cluster_wait();
    if (trace && threadIdx.x == 0) trace[7] = static_cast<long long>(ptx::globaltimer_ns());
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
        // CTAs per SM aimed at: two for small M; one for M > 32, where half as many splits halve the reduce-scatter
        // and a single CTA can afford a ring twice as deep (B200FP8_SKINNY_CTAS_PER_SM overrides)
        static const int fill_env = [] { const char* v = getenv("B200FP8_SKINNY_CTAS_PER_SM"); return v ? atoi(v) : 0; }();
        const int fill = fill_env > 0 ? fill_env : (mp >= 64 ? 1 : 2);
        s = (fill * sm_count) / n_tiles;
        if (s < 1) s = (2 * sm_count) / n_tiles;
        if (s < 1) s = 1;
        // clusters of 8 CTAs pack badly into the GPCs: with more than 8 of them some wait for a second round
        // (K = 8192, N = 2048: M = 128 17 us with 8 splits, 10.8 us with 4; M = 16 11.8 us against 7.6 us)
        if (s > 4 && n_tiles > 8) s = 4;
        // a split wants k-blocks of its own: with too few, the reduce-scatter of one more partial tile costs more than
        // the shorter stream saves.  Eight for M > 64, whose partial tiles are large (128 x 4096 x 1024: 6.8 us with 4
        // splits against 7.4 with 8); four for smaller M once there are N tiles enough to occupy the GPU anyway
        // (16 x 1024 x 4096: 3.7 us with 2 against 4.0 with 4; with 8-16 N tiles more splits still win: 1 x 2048 x 2048
        // 3.5 us with 4 against 4.0 with 2, 48 x 2048 x 2048 4.5 with 4 against 5.2 with 2)
        if (mp > 64 || n_tiles >= 32) {
            const int own = mp > 64 ? 8 : 4;
            int by_k = 2;
            while (2 * kb_total >= 3 * by_k * own) by_k *= 2;      // kb_total / own rounded to the nearest power of two
            if (s > by_k) s = by_k;
        }
    }
    if (s > kSkinnyMaxSplits) s = kSkinnyMaxSplits;
    if (s > kb_total) s = kb_total;
    int per = (kb_total + s - 1) / s;
    s = (kb_total + per - 1) / per;          // no empty split
    if (split_k <= 0) {
        // the planner's own choice is a power of two: clusters of 3, 5, 6 or 7 CTAs place badly
        // (16 x 1536 x 6144: 7.8 us with 3 splits against 4.7 with 2 or 4)
        while (s & (s - 1)) {
            int p = 1;
            while (2 * p <= s) p *= 2;
            per = (kb_total + p - 1) / p;
            s = (kb_total + per - 1) / per;
            if (s & (s - 1)) --s;            // e.g. 9 k-blocks: 4 splits of 3 leave 3 splits; go on from 2
        }
        per = (kb_total + s - 1) / s;
    }
    *splits = s;
    *kb_per_split = per;
    int st = depth;
    if (st <= 0) {
        const int stage_bytes = (kSkinnyTileN + mp) * kBlockK;
        // two CTAs per SM share its shared memory; a grid that fits one CTA per SM gets all of it
        const int budget = (static_cast<long long>(n_tiles) * s <= sm_count ? 216 : 108) * 1024;
        st = budget / stage_bytes;
        if (st > 8) st = 8;
        if (st < 2) st = 2;
    }
    *stages = st;
}

template <int MP, int THREADS>
cudaError_t launch_skinny_mp(const CUtensorMap& tb, const CUtensorMap& ta, const SkinnyArgs& args, int n_tiles,
                             cudaStream_t stream) {
    using L = SkinnySmem<MP>;
    auto kernel = gemm_fp8_skinny_kernel<MP, THREADS>;
    static int attr_bytes[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int bytes = L::dynamic_bytes(args.stages);
    if (attr_bytes[dev] < bytes) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        attr_bytes[dev] = bytes;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(n_tiles), static_cast<unsigned>(args.splits), 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(args.splits);
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see griddep_wait in the kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = args.pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, tb, ta, args);
}

inline cudaError_t launch_skinny(int sm_count, int* status, SkinnyEncodeFn enc, int m, int k, int n, const void* a,
                                 long long lda, const void* b, long long ldb, float* c, long long ldc, int a_dtype,
                                 int b_dtype, int depth, int split_k, const Epilogue* epi, cudaStream_t stream,
                                 const int* ell_col_ind = nullptr, int ell_k_small = 0, long long* trace = nullptr, int pdl = 0) {
    // With ell_col_ind the large operand B is in blocked-ELL form: `k` is the width of its compact values matrix
    // (blocks per row x 128) and ell_k_small the K of the small operand A.
    const int mp = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    const int n_tiles = (n + kSkinnyTileN - 1) / kSkinnyTileN;
    if (n_tiles > 65535 * 32) return cudaErrorInvalidValue;
    SkinnyArgs args{};
    skinny_plan(sm_count, n, k, mp, depth, split_k, &args.splits, &args.kb_per_split, &args.stages);
    args.M = m; args.N = n; args.K = k;
    args.kb_total = (k + kBlockK - 1) / kBlockK;
    args.vec_store = ((ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(c) % 16) == 0) ? 1 : 0;
    args.idesc = make_idesc_f8(b_dtype, a_dtype, 128, mp);   // swapped: B feeds the UMMA A operand
    args.C = c; args.ldc = ldc;
    args.status = status;
    if (epi) args.epi = *epi;
    args.trace = trace;
    args.pdl = pdl;
    // measured at N = K = 8192 in graphs of back-to-back launches: 8 blocks (128 KiB per CTA) take 0.4-0.5 us off
    // M <= 16, 0.2 us off M = 64, nothing off M = 128; 16 blocks are no better (B200FP8_SKINNY_L2_PREFETCH overrides)
    static const int prefetch_env = [] { const char* v = getenv("B200FP8_SKINNY_L2_PREFETCH"); return v ? atoi(v) : 8; }();
    args.l2_prefetch = pdl ? prefetch_env : 0;
    if (ell_col_ind) {
        args.ell_col_ind = ell_col_ind;
        args.ell_oob_a = (ell_k_small + kBlockK - 1) / kBlockK * kBlockK;
        args.ell_oob_b = args.kb_total * kBlockK;
    }
    CUtensorMap tb, ta;
    cudaError_t e;
    if ((e = skinny_encode(enc, &tb, b, k, n, ldb, kSkinnyTileN)) != cudaSuccess) return e;
    if ((e = skinny_encode(enc, &ta, a, ell_col_ind ? ell_k_small : k, m, lda, mp)) != cudaSuccess) return e;
    static const int threads_env = [] { const char* v = getenv("B200FP8_SKINNY_THREADS"); return v ? atoi(v) : 0; }();
    // the wide launch needs the SM to itself (one CTA per SM) and only pays when there is something to exchange
    const bool one_per_sm = static_cast<long long>(n_tiles) * args.splits <= sm_count;
    int threads = (mp >= 64 && args.splits > 1 && one_per_sm) ? kSkinnyThreadsWide : kSkinnyThreads;
    if (threads_env == 192 || (threads_env == 512 && one_per_sm) || (threads_env == 1024 && one_per_sm)) threads = threads_env;
    switch (mp) {
        case 16: return launch_skinny_mp<16, kSkinnyThreads>(tb, ta, args, n_tiles, stream);
        case 32: return launch_skinny_mp<32, kSkinnyThreads>(tb, ta, args, n_tiles, stream);
        case 64:
            if (threads == 1024) return launch_skinny_mp<64, 1024>(tb, ta, args, n_tiles, stream);
            if (threads == 512) return launch_skinny_mp<64, 512>(tb, ta, args, n_tiles, stream);
            return launch_skinny_mp<64, kSkinnyThreads>(tb, ta, args, n_tiles, stream);
        default:
            if (threads == 1024) return launch_skinny_mp<128, 1024>(tb, ta, args, n_tiles, stream);
            if (threads == 512) return launch_skinny_mp<128, 512>(tb, ta, args, n_tiles, stream);
            return launch_skinny_mp<128, kSkinnyThreads>(tb, ta, args, n_tiles, stream);
    }
}

}  // namespace b200fp8
