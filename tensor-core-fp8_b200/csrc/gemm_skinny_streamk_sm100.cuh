// Skinny (decode-shaped) FP8 GEMM for sm_100a, stream-K form: M <= 128 rows of A against a large B.
// The work is streaming B[N][K] once from HBM; what the clustered split-K kernel (gemm_skinny_sm100.cuh)
// loses around that stream -- SMs without a CTA, splits of a tile that finish at different times, a
// reduce-scatter over the cluster network and two cluster barriers, none of it overlapping anything --
// is what this kernel is organised to avoid:
//
//   * one persistent CTA per SM and one linear space of work units, unit = (N tile of 128 rows of B,
//     k-block of 128 bytes).  CTA c owns the units [c U / G, (c+1) U / G): every SM streams the same number
//     of bytes (+-1 block), whatever N and K are, and the TMA ring never drains between tiles;
//   * swap-AB as before: the 128 rows of B ride the UMMA M axis, A's rows padded to MP in {16,32,64,128}
//     (TMA zero fill) the N axis, the accumulator is C^T (TMEM lane = n, column = m);
//   * a CTA's range cuts through at most two tiles (more, with whole tiles between, when U / G exceeds a
//     tile's K).  Each piece ("segment") gets one of two TMEM accumulator slots, so the epilogue of a
//     segment runs under the stream of the next one;
//   * a segment that does not start its tile parks its partial sums in a scratch slot in global memory
//     (L2) and raises a flag; the CTA that holds the START of a tile finishes it: it adds the parked
//     partials to its own accumulator in ascending K order -- a fixed order, so the result does not depend
//     on timing -- and writes C.  A CTA parks first and finishes last, and finishers only ever wait for
//     CTAs that were dispatched before them (the unit space is walked from the highest block index down),
//     so the waits cannot form a cycle; they are bounded all the same;
//   * flags are consumed and cleared by the finisher, so a launch leaves them as it found them (zero) and a
//     captured graph can be replayed without a memset node between the kernels.
//
// Same operator contract as the other kernels (reference: gemm::GEMM, GEMM/include/gemm.cuh:12-55; the
// reference's kernels write nothing at all for M < 128, GEMM/src/gemm.cu:45-47).
#pragma once
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "gemm_sm100.cuh"
#include "gemm_skinny_sm100.cuh"

namespace b200fp8 {

constexpr int kStreamKThreads = 192;        // warp 0 TMA producer, warp 1 MMA issue, warps 2-5 epilogue
constexpr int kStreamKMaxStages = 12;
constexpr int kStreamKParkRows = 64;        // rows of C staged at a time for the row-wise stores

struct StreamKArgs {
    int M, N, K;
    int kb_total;            // ceil(K / 128)
    int n_tiles;             // ceil(N / 128)
    long long units;         // n_tiles * kb_total
    int stages;
    int vec_store;           // 1: C rows are 16-byte aligned (ldc % 4 == 0 and C % 16 == 0)
    int l2_prefetch;         // k-blocks of the CTA's first units prefetched into L2 before the grid dependency wait
    uint32_t idesc;
    float* C;
    long long ldc;
    int* status;
    float4* scratch;         // [gridDim.x][MP / 4][128] parked partial tiles (float4 = four consecutive m of one n)
    unsigned int* flags;     // [gridDim.x]: 0 at launch; 1 = the CTA's partial is parked; cleared by the finisher
    // blocked-ELL form of the LARGE operand B, as in SkinnyArgs
    const int* ell_col_ind;
    int ell_oob_a, ell_oob_b;
    long long* trace;        // diagnostics build only: eight globaltimer stamps per CTA (nullptr = off)
    Epilogue epi;
};

template <int MP>
struct StreamKSmem {
    static constexpr int kBBytes = kSkinnyTileN * kBlockK;
    static constexpr int kABytes = MP * kBlockK;
    static constexpr int kStageBytes = kBBytes + kABytes;
    static constexpr int kParkRows = MP < kStreamKParkRows ? MP : kStreamKParkRows;
    static constexpr int kParkBytes = kParkRows * kSkinnyTileN * 4;
    static constexpr int kCols = MP < 32 ? 32 : MP;            // TMEM columns of one accumulator slot
    static constexpr int kTmemCols = 2 * kCols;                // two slots: 64, 64, 128 or 256
    static constexpr int kNumBars = 2 * kStreamKMaxStages + 5; // full[], empty[], tfull[2], tempty[2], fix
    static constexpr int kTailBytes = 8 * kNumBars + 32;
    __host__ __device__ static constexpr int park_off(int stages) { return stages * kStageBytes; }
    __host__ __device__ static constexpr int bar_off(int stages) { return park_off(stages) + kParkBytes; }
    __host__ __device__ static constexpr int dynamic_bytes(int stages) { return bar_off(stages) + kTailBytes + 1024; }
    static constexpr int max_stages(int budget_bytes) {
        return (budget_bytes - 1024 - kTailBytes - kParkBytes) / kStageBytes;
    }
};

namespace ptx {
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// barrier among the 128 epilogue threads only (barrier 0 is __syncthreads)
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// OR-reduction of a predicate over the 128 epilogue threads; every one of them gets the same answer (and they meet
// as at a barrier), so a decision to leave the loop is taken by all of them or by none
__device__ __forceinline__ bool epilogue_any(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "barrier.cta.red.or.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}"
        : "=r"(r) : "r"(static_cast<uint32_t>(pred)) : "memory");
    return r != 0;
}
// untiled bulk copy global -> this CTA's shared memory, completion (byte count) on this CTA's mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// orders this thread's earlier generic-proxy accesses before its later async-proxy (bulk copy) accesses
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// L2 prefetch of a tensor box: a hint without architectural effect on the data
__device__ __forceinline__ void tma_prefetch_2d(const void* tmap, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
                 ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y) : "memory");
}
}  // namespace ptx

template <int MP>
__global__ void __launch_bounds__(kStreamKThreads, 1)
gemm_fp8_skinny_streamk_kernel(const __grid_constant__ CUtensorMap tmap_b,   // B[N][K], box 128 rows
                               const __grid_constant__ CUtensorMap tmap_a,   // A[M][K], box MP rows
                               const StreamKArgs args)
{
    using L = StreamKSmem<MP>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
    const int stages = args.stages;
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // provably warp-uniform
    const int lane = threadIdx.x & 31;

    const uint32_t bar_full = smem_base + L::bar_off(stages);
    const uint32_t bar_empty = bar_full + 8 * kStreamKMaxStages;
    const uint32_t bar_tfull = bar_empty + 8 * kStreamKMaxStages;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t bar_fix = bar_tempty + 16;          // bulk copies of parked partials into the idle ring
    const int misc_off = L::bar_off(stages) + 8 * L::kNumBars;
    const uint32_t tmem_slot = smem_base + misc_off;
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + misc_off + 8);

    long long* trace = (kDiagnostics && args.trace) ? args.trace + 8ll * blockIdx.x : nullptr;   // diagnostics build only
    if (trace && threadIdx.x == 0) trace[0] = static_cast<long long>(ptx::globaltimer_ns());
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, 4);          // one arrival per epilogue warp
        }
        ptx::mbar_init(bar_fix, 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(tmem_slot, L::kTmemCols);
        ptx::tmem_relinquish<1>();
    }

    // this CTA's units: the space is handed out from the highest block index down, so that the CTAs a finisher
    // waits for (those that hold the rest of its tile: higher unit numbers) have lower block indices
    const long long G = gridDim.x;
    const long long c = G - 1 - blockIdx.x;
    const long long u_begin = c * args.units / G;
    const long long u_end = (c + 1) * args.units / G;
    const int kbt = args.kb_total;

    if (warp == 0 && args.l2_prefetch > 0 && args.ell_col_ind == nullptr) {
        // The first blocks of B this CTA will stream, requested into L2 before the wait below: a prefetch changes no
        // data anywhere (L2 is the point of coherence; a line the previous kernel still writes stays correct), it
        // only starts the first HBM round trip while the previous kernel of the stream drains
        if (ptx::elect_one()) {
            long long u = u_begin;
            for (int i = 0; i < args.l2_prefetch && u < u_end; ++i, ++u) {
                const int tile = static_cast<int>(u / kbt);
                const int kb = static_cast<int>(u - static_cast<long long>(tile) * kbt);
                ptx::tma_prefetch_2d(&tmap_b, kb * kBlockK, tile * kSkinnyTileN);
            }
        }
        __syncwarp();
    }

    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;
    // Everything above touched only this CTA's own resources (and hinted L2) and may overlap the previous kernel's
    // tail; global memory is read or written only after the grids before this one are complete.
    ptx::griddep_wait();
    ptx::griddep_launch_dependents();
    if (trace && threadIdx.x == 0) trace[1] = static_cast<long long>(ptx::globaltimer_ns());

    if (warp == 0) {
        // ---------------- TMA producer: one uninterrupted stream over all of the CTA's units ----------------
        int s = 0;
        uint32_t ph = 0;
        int issued = 0;
        bool ok = true;
        for (long long u = u_begin; u < u_end && ok;) {
            const int tile = static_cast<int>(u / kbt);
            const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * kbt);
            const int kb1 = static_cast<int>(min(static_cast<long long>(kbt), kb0 + (u_end - u)));
            const int n0 = tile * kSkinnyTileN;
            // blocked-ELL B: lane l holds the column block of k-block (chunk base + l); the next 32 are prefetched
            const int* ell_row = nullptr;
            int ell_cur = -1, ell_nxt = -1;
            if (args.ell_col_ind != nullptr) {
                ell_row = args.ell_col_ind + static_cast<long long>(tile) * kbt;
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
            u += kb1 - kb0;
        }
        if (!ok) {
            // leave no copy in flight into this CTA's shared memory: wait (bounded) for the slots armed last
            const int pending = issued < stages ? issued : stages;
            for (int i = 0; i < pending; ++i) {
                if (s == 0) { s = stages; ph ^= 1u; }
                --s;
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(bar_full + 8 * s, ph) && ptx::globaltimer_ns() - t0 < kWaitLimitNs) {}
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue: segment i accumulates into TMEM slot i & 1 ----------------
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        int seg = 0;
        for (long long u = u_begin; u < u_end && ok; ++seg) {
            const int tile = static_cast<int>(u / kbt);
            const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * kbt);
            const int kb1 = static_cast<int>(min(static_cast<long long>(kbt), kb0 + (u_end - u)));
            const int slot = seg & 1;
            if (!wait_bounded(bar_tempty + 8 * slot, static_cast<uint32_t>((seg >> 1) & 1) ^ 1u, abort_flag, false)) {
                record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
                break;
            }
            ptx::tc_fence_after();
            const uint32_t d_tmem = tmem_base + slot * L::kCols;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!wait_bounded(bar_full + 8 * s, ph, abort_flag, false)) {
                    record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (trace && u == u_begin && kb == kb0 && lane == 0) trace[2] = static_cast<long long>(ptx::globaltimer_ns());
                const uint32_t b_src = smem_base + s * L::kStageBytes;
                const uint64_t adesc = ptx::umma_desc_k128(b_src);                 // 128 rows of B
                const uint64_t bdesc = ptx::umma_desc_k128(b_src + L::kBBytes);    // MP rows of A
                if (ptx::elect_one()) {
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k)
                        ptx::umma_f8<1>(d_tmem, adesc + 2 * k, bdesc + 2 * k, args.idesc, (kb > kb0) || (k > 0));
                    ptx::umma_commit(bar_empty + 8 * s);
                }
                __syncwarp();
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
            if (ok && ptx::elect_one()) ptx::umma_commit(bar_tfull + 8 * slot);
            __syncwarp();
            u += kb1 - kb0;
        }
        if (trace && lane == 0) trace[3] = static_cast<long long>(ptx::globaltimer_ns());
    } else {
        // ---------------- epilogue: 128 threads, thread = one column n of C (one TMEM lane) ----------------
        const int q = warp & 3;                                  // TMEM lane quarter this warp may read
        const int n_local = q * 32 + lane;
        const int tid = (warp - 2) * 32 + lane;                  // 0..127 among the epilogue threads
        float* park = reinterpret_cast<float*>(smem_gen + L::park_off(stages));
        const uint32_t park_addr = smem_base + L::park_off(stages);
        float epi_alpha = 1.0f, epi_dscale = 1.0f, epi_amax = 0.0f;
        if (args.epi.active) {
            epi_alpha = args.epi.alpha;
            if (args.epi.a_scale) epi_alpha *= *args.epi.a_scale;
            if (args.epi.b_scale) epi_alpha *= *args.epi.b_scale;
            if (args.epi.d_scale) epi_dscale = *args.epi.d_scale;
        }
        constexpr int kGroups = MP / 4;                          // float4 groups (four consecutive m) per column
        const int groups = min(kGroups, (args.M + 3) >> 2);
        int seg = 0;
        for (long long u = u_begin; u < u_end; ++seg) {
            const int tile = static_cast<int>(u / kbt);
            const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * kbt);
            const int kb1 = static_cast<int>(min(static_cast<long long>(kbt), kb0 + (u_end - u)));
            const int slot = seg & 1;
            const int n0 = tile * kSkinnyTileN;
            u += kb1 - kb0;
            const bool got = wait_bounded(bar_tfull + 8 * slot, static_cast<uint32_t>((seg >> 1) & 1), abort_flag, false);
            if (!got) record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
            if (ptx::epilogue_any(!got)) break;                   // all 128 threads leave together: the barriers below stay whole
            ptx::tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + slot * L::kCols;
            auto release_slot = [&]() {                          // this warp's accumulator lanes are in registers
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_tempty + 8 * slot);
            };

            if (kb0 != 0) {
                // ---- not the start of its tile: park the partial sums for the tile's finisher ----
                float4* dst = args.scratch + (c * kGroups) * kSkinnyTileN + n_local;
#pragma unroll
                for (int ch = 0; ch < MP / 16; ++ch) {
                    if (ch * 16 < args.M) {
                        uint32_t v[16];
                        ptx::tmem_ld_32x16(t_addr + ch * 16, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (ch * 4 + j < groups)
                                __stcg(dst + (ch * 4 + j) * kSkinnyTileN,
                                       make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                   __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                    }
                }
                release_slot();
                __threadfence();
                ptx::epilogue_barrier();
                if (tid == 0) ptx::st_release_gpu(args.flags + c, 1u);
                continue;
            }

            // ---- start of a tile: this CTA finishes it.  The rest of the tile's K range (if any) belongs to the
            //      CTAs c+1, c+2, ... (lower block indices); wait for their parked partials ----
            int peers = 0;
            if (kb1 != kbt) {
                const long long tile_end = (static_cast<long long>(tile) + 1) * kbt;
                while (c + 1 + peers < G && (c + 1 + peers) * args.units / G < tile_end) ++peers;
                bool seen = true;
                for (int p = 0; p < peers && seen; ++p) {
                    const unsigned int* f = args.flags + c + 1 + p;
                    uint64_t t0 = 0;
                    uint32_t spins = 0;
                    while (ptx::ld_acquire_gpu(f) == 0u) {
                        if ((++spins & 0x3Fu) == 0) {
                            const uint64_t now = ptx::globaltimer_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > kWaitLimitNs || *abort_flag) { seen = false; break; }
                        }
                    }
                }
                if (!seen) record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
                if (ptx::epilogue_any(!seen)) {
                    release_slot();
                    break;
                }
            }
            if (trace && u >= u_end && tid == 0) trace[4] = static_cast<long long>(ptx::globaltimer_ns());
            const float4* src = args.scratch + ((c + 1) * kGroups) * kSkinnyTileN + n_local;
            // The parked partials come over as bulk copies into the ring, which is idle by now (a tile with peers is
            // the CTA's last segment and all of its MMAs are complete): one thread issues, the copy engine moves the
            // bytes at full rate, and the additions read shared memory.  (Element-wise loads from L2 are latency-bound:
            // a handful in flight per thread.)  Falls back to loads when the partials of one pass do not fit.
            constexpr int kGroupBytes = kSkinnyTileN * 16;          // one float4 group of all 128 columns
            const bool bulk = peers > 0 && peers * (L::kParkRows / 4) * kGroupBytes <= stages * L::kStageBytes;
            uint32_t fix_phase = 0;
            bool fix_ok = true;
#pragma unroll 1
            for (int half = 0; half < MP / L::kParkRows; ++half) {
                const int m_half = half * L::kParkRows;
                if (m_half >= args.M) break;
                const int g_half = m_half >> 2;
                const int g_cnt = min(groups - g_half, L::kParkRows / 4);
                if (bulk) {
                    if (tid == 0) {
                        ptx::fence_proxy_async_all();
                        ptx::mbar_arrive_expect_tx(bar_fix, static_cast<uint32_t>(peers * g_cnt * kGroupBytes));
                        for (int p = 0; p < peers; ++p)
                            ptx::bulk_load(smem_base + static_cast<uint32_t>(p * g_cnt * kGroupBytes),
                                           args.scratch + ((c + 1 + p) * kGroups + g_half) * kSkinnyTileN,
                                           static_cast<uint32_t>(g_cnt * kGroupBytes), bar_fix);
                    }
                    const bool landed = wait_bounded(bar_fix, fix_phase, abort_flag, false);
                    fix_phase ^= 1u;
                    if (!landed) record_failure(args.status, abort_flag, kStatusSkinnyTimeout);
                    if (ptx::epilogue_any(!landed)) { fix_ok = false; break; }
                    if (trace && half == 0 && tid == 0) trace[5] = static_cast<long long>(ptx::globaltimer_ns());
                }
#pragma unroll
                for (int ch = 0; ch < L::kParkRows / 16; ++ch) {
                    const int m_ch = m_half + ch * 16;
                    if (m_ch < args.M) {
                        uint32_t v[16];
                        ptx::tmem_ld_32x16(t_addr + m_ch, v);
                        ptx::tmem_ld_wait();
                        for (int p = 0; p < peers; ++p) {         // ascending K: the fixed summation order
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int g4 = (m_ch >> 2) + j;
                                if (g4 < groups) {
                                    float4 w;
                                    if (bulk) w = ld_local_f4(smem_base + static_cast<uint32_t>(((p * g_cnt + g4 - g_half) * kSkinnyTileN + n_local) * 16));
                                    else w = __ldcg(src + (static_cast<long long>(p) * kGroups + g4) * kSkinnyTileN);
                                    v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + w.x);
                                    v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + w.y);
                                    v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + w.z);
                                    v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + w.w);
                                }
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (m_ch + j < args.M) park[(ch * 16 + j) * kSkinnyTileN + n_local] = __uint_as_float(v[j]);
                    }
                }
                if (m_half + L::kParkRows >= args.M || half + 1 == MP / L::kParkRows) release_slot();
                ptx::epilogue_barrier();
                // row-wise stores: one instruction writes 512 consecutive bytes of one row of C
                const int rows = min(L::kParkRows, args.M - m_half);
                const int items = rows * (kSkinnyTileN / 4);
                for (int i = tid; i < items; i += 128) {
                    const int m = m_half + i / (kSkinnyTileN / 4);
                    const int cg = i % (kSkinnyTileN / 4);
                    const float4 acc = ld_local_f4(park_addr + static_cast<uint32_t>(((m - m_half) * kSkinnyTileN + cg * 4) * 4));
                    const int n = n0 + cg * 4;
                    const long long idx = static_cast<long long>(m) * args.ldc + n;
                    float* dst = args.C + idx;
                    if (args.epi.active) {
                        if (n < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx, m, n, acc.x, epi_amax);
                        if (n + 1 < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx + 1, m, n + 1, acc.y, epi_amax);
                        if (n + 2 < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx + 2, m, n + 2, acc.z, epi_amax);
                        if (n + 3 < args.N) skinny_store_epi(args, epi_alpha, epi_dscale, idx + 3, m, n + 3, acc.w, epi_amax);
                    } else if (args.vec_store && n + 3 < args.N) {
                        *reinterpret_cast<float4*>(dst) = acc;
                    } else {
                        if (n < args.N) dst[0] = acc.x;
                        if (n + 1 < args.N) dst[1] = acc.y;
                        if (n + 2 < args.N) dst[2] = acc.z;
                        if (n + 3 < args.N) dst[3] = acc.w;
                    }
                }
                ptx::epilogue_barrier();                          // the staging rows are free again
            }
            if (!fix_ok) {
                release_slot();
                break;
            }
            // every epilogue thread has read the parked partials (barrier above): hand the flags back as zero
            for (int p = tid; p < peers; p += 128) args.flags[c + 1 + p] = 0u;
        }
        __syncwarp();
        if (args.epi.amax != nullptr) amax_merge_warp(args.epi.amax, epi_amax);
        if (trace && tid == 0) trace[6] = static_cast<long long>(ptx::globaltimer_ns());
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem_base, L::kTmemCols);
    }
    if (trace && threadIdx.x == 0) trace[7] = static_cast<long long>(ptx::globaltimer_ns());
}

// Scratch memory of the stream-K kernel on one device: a ring of slots, one per launch in flight.  Each slot
// holds one parked partial tile per CTA and one flag per CTA.  Launches on ONE stream may share a slot (a launch
// starts only after the previous one has completed); the ring covers launches that overlap on different streams.
struct StreamKWorkspace {
    static constexpr int kSlots = 4;
    float4* scratch[kSlots] = {};
    unsigned int* flags[kSlots] = {};
    unsigned int next = 0;
    int max_ctas = 0;
    static size_t scratch_bytes(int ctas) { return static_cast<size_t>(ctas) * kSkinnyMaxM * kSkinnyTileN * sizeof(float); }
};

// Grid size (CTAs) of the stream-K kernel: every SM, unless that would cut tiles into so many pieces that the
// finisher's serial additions cost more than the missing SMs (at most 8 pieces per tile for small M, 4 for M > 32)
inline int streamk_grid(int sm_count, int n_tiles, int kb_total, int mp, int split_k) {
    static const int grid_env = [] { const char* v = getenv("B200FP8_SKINNY_GRID"); return v ? atoi(v) : 0; }();
    const long long units = static_cast<long long>(n_tiles) * kb_total;
    long long g = sm_count;
    const long long pieces = split_k > 0 ? split_k : (mp >= 64 ? 4 : 8);
    if (g > static_cast<long long>(n_tiles) * pieces) g = static_cast<long long>(n_tiles) * pieces;
    if (grid_env > 0 && grid_env < g) g = grid_env;
    if (g > units) g = units;
    return static_cast<int>(g < 1 ? 1 : g);
}

template <int MP>
cudaError_t launch_streamk_mp(const CUtensorMap& tb, const CUtensorMap& ta, StreamKArgs& args, int grid, int depth,
                              int pdl, cudaStream_t stream) {
    using L = StreamKSmem<MP>;
    auto kernel = gemm_fp8_skinny_streamk_kernel<MP>;
    static int attr_bytes[64] = {};
    static const int stages_env = [] { const char* v = getenv("B200FP8_SKINNY_STAGES"); return v ? atoi(v) : 0; }();
    int st = L::max_stages(227 * 1024);
    if (st > kStreamKMaxStages) st = kStreamKMaxStages;
    if (stages_env >= 2 && stages_env < st) st = stages_env;
    if (depth > 0 && depth < st) st = depth;
    args.stages = st;
    int dev = 0;
    cudaGetDevice(&dev);
    const int bytes = L::dynamic_bytes(st);
    if (attr_bytes[dev] < bytes) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        attr_bytes[dev] = bytes;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(kStreamKThreads, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see griddep_wait in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, tb, ta, args);
}

// `scratch` / `flags`: one workspace slot, sized for at least `sm_count` CTAs (see StreamKWorkspace).
inline cudaError_t launch_skinny_streamk(int sm_count, int* status, float4* scratch, unsigned int* flags,
                                         SkinnyEncodeFn enc, int m, int k, int n, const void* a, long long lda,
                                         const void* b, long long ldb, float* c, long long ldc, int a_dtype, int b_dtype,
                                         int depth, int split_k, const Epilogue* epi, cudaStream_t stream,
                                         const int* ell_col_ind = nullptr, int ell_k_small = 0, long long* trace = nullptr,
                                         int pdl = 0) {
    // With ell_col_ind the large operand B is in blocked-ELL form: `k` is the width of its compact values matrix
    // (blocks per row x 128) and ell_k_small the K of the small operand A.
    static const int prefetch_env = [] { const char* v = getenv("B200FP8_SKINNY_L2_PREFETCH"); return v ? atoi(v) : 8; }();
    const int mp = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    const int n_tiles = (n + kSkinnyTileN - 1) / kSkinnyTileN;
    if (n_tiles > 65535 * 32) return cudaErrorInvalidValue;
    StreamKArgs args{};
    args.M = m; args.N = n; args.K = k;
    args.kb_total = (k + kBlockK - 1) / kBlockK;
    args.n_tiles = n_tiles;
    args.units = static_cast<long long>(n_tiles) * args.kb_total;
    args.vec_store = ((ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(c) % 16) == 0) ? 1 : 0;
    args.l2_prefetch = pdl ? prefetch_env : 0;
    args.idesc = make_idesc_f8(b_dtype, a_dtype, 128, mp);   // swapped: B feeds the UMMA A operand
    args.C = c; args.ldc = ldc;
    args.status = status;
    args.scratch = scratch;
    args.flags = flags;
    if (epi) args.epi = *epi;
    args.trace = trace;
    if (ell_col_ind) {
        args.ell_col_ind = ell_col_ind;
        args.ell_oob_a = (ell_k_small + kBlockK - 1) / kBlockK * kBlockK;
        args.ell_oob_b = args.kb_total * kBlockK;
    }
    const int grid = streamk_grid(sm_count, n_tiles, args.kb_total, mp, split_k);
    CUtensorMap tb, ta;
    cudaError_t e;
    if ((e = skinny_encode(enc, &tb, b, k, n, ldb, kSkinnyTileN)) != cudaSuccess) return e;
    if ((e = skinny_encode(enc, &ta, a, ell_col_ind ? ell_k_small : k, m, lda, mp)) != cudaSuccess) return e;
    switch (mp) {
        case 16: return launch_streamk_mp<16>(tb, ta, args, grid, depth, pdl, stream);
        case 32: return launch_streamk_mp<32>(tb, ta, args, grid, depth, pdl, stream);
        case 64: return launch_streamk_mp<64>(tb, ta, args, grid, depth, pdl, stream);
        default: return launch_streamk_mp<128>(tb, ta, args, grid, depth, pdl, stream);
    }
}

}  // namespace b200fp8
