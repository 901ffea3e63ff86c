// Main FP8 GEMM kernel for sm_100a: C[M][N] (FP32, row-major) = A[M][K] * B[N][K]^T with
// A and B stored as 8-bit floats, K contiguous in both ("row-col" layout of the reference
// operator gemm::GEMM, GEMM/include/gemm.cuh:12-55).  It replaces the reference's
// cp.async + mma.sync.m16n8k32 kernels (GEMM/src/gemm.cu:29-262 and its copies).
//
// Structure (one persistent CTA, or CTA pair, per SM):
//   warp 0      TMA producer: A and B k-blocks (128 bytes of K per block, 128-byte swizzle)
//               into a STAGES-deep shared-memory ring guarded by full/empty mbarriers
//   warp 1      TMEM allocation; one lane issues tcgen05.mma kind::f8f6f4 (four K=32
//               instructions per k-block) into one of two TMEM accumulator buffers and
//               commits to the ring's empty barriers / the accumulator's full barrier
//   warps 2-9   epilogue, two groups of four warps (a warp may only read its own quarter of the
//               TMEM lanes): tcgen05.ld 32 rows x 32 columns at a time, software-pipelined against
//               the stores, staged through swizzled shared memory, TMA-stored as 32x32 FP32 boxes
//               (hardware clips ragged M/N edges); runs concurrently with the next tile's main
//               loop (two TMEM accumulator slots).  With one accumulator per tile the groups
//               split its columns; with two (NACC == 2) each group drains one of them
// CTAS == 2 pairs two CTAs of a cluster on a 256 x BN tile (cta_group::2): each CTA loads
// its own 128 rows of A and its own half of the B tile (no multicast), the leader CTA
// issues the MMAs for both, and each CTA drains its own 128 accumulator rows.
// NACC == 2 widens the tile to 256 x (2*BN): both TMEM accumulator slots belong to the same
// tile (columns [0,BN) and [BN,2BN)), every A k-block feeds two MMAs, and shared-memory,
// L2 and HBM traffic per flop drop by a quarter; the price is that the epilogue of a tile
// overlaps only the head of the next tile's main loop instead of all of it.  The wide tile
// wins on large problems, where the GPU runs at its power limit and energy per flop
// decides the clock.
//
// Also in this kernel: tail balancing (a last round that would keep at most half of the CTAs busy
// runs as half-width work items), tile pacing (leaders briefly wait for each other before a new
// tile so that panels are shared through L2), the scaled epilogue (alpha, beta, scale pointers,
// BF16/FP16 output) and, for N-sharded multi-GPU runs, the fused all-gather (finished boxes are
// also stored into every peer's C, by unicast stores or one multimem store).
//
// Also: a blocked-ELL sparse A for the one-CTA variants (one table lookup per k-block in the producer), a
// plain-store epilogue for C matrices TMA cannot write (transposed through the staging box: coalesced rows), and
// programmatic dependent launch (set-up before griddepcontrol.wait, global memory only after it).
//
// Every wait on an mbarrier is bounded: after about two seconds the waiting warp records a
// code in the device status word, raises a CTA-wide abort flag and leaves its loop, so a
// broken pipeline ends the kernel instead of hanging the GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include "ptx_sm100.cuh"

namespace b200fp8 {

// Extended epilogue:
//     t = act(alpha * sa * sb * ra[m] * rb[n] * (A B^T) + beta * D + bias[n])      amax = max |t| over the valid part of D
//     D = convert(sd * t)                                                          D in FP32, BF16, FP16, E4M3 or E5M2
// ra / rb are optional vectors of per-row scales of A (M values) and of B (N values): the "outer vector" scaling of
// cuBLASLt; act is none, ReLU or GELU (erf or tanh form), applied after the bias as cuBLASLt's fused epilogues do
// (the knobs of the reference's cuBLASLt comparator, GEMM/src/cublas.cu:37-53: alpha, beta, scale pointers;
// 8-bit outputs are rounded to nearest even and saturate to the largest finite value, like the toolkit's
// host conversions that the reference uses for its inputs).  The plain operator (alpha = 1, beta = 0, FP32)
// leaves `active` at 0 and pays nothing for it.
struct Epilogue {
    int active;            // 0: plain FP32 store of the accumulator
    int out_dtype;         // 0 FP32, 1 BF16, 2 FP16, 3 E4M3, 4 E5M2
    float alpha, beta;
    const float* a_scale;  // optional device scalars multiplied into alpha
    const float* b_scale;
    const float* d_scale;  // optional device scalar applied just before the conversion to out_dtype
    float* amax;           // optional device float (zero at launch): receives max |t| by atomic max; NaNs are ignored
    const void* bias;      // optional device vector of N values added to every row
    int bias_dtype;        // 0 FP32, 1 BF16, 2 FP16
    const float* a_row_scale;   // optional device vector of M factors, one per row of A (= row of D)
    const float* b_row_scale;   // optional device vector of N factors, one per row of B (= column of D)
    int activation;        // 0 none, 1 ReLU, 2 GELU 0.5 t (1 + erf(t / sqrt 2)), 3 GELU 0.5 t (1 + tanh(sqrt(2/pi) (t + 0.044715 t^3)))
};

// The activations.  Code size matters more than instruction count here: the tile kernels unroll the epilogue over 32
// accumulator registers at three places, every instruction of it runs a handful of times per launch, and a one-tile
// launch pays an instruction-cache miss for every line it touches (ReLU written as one branch of a per-element
// switch next to an inlined erff doubled the time of 2048^3; erff behind a call cost 10 us there).  So: one loop per
// activation, and branch-free formulas of a dozen instructions.
__device__ __forceinline__ float relu(float t) { return t > 0.0f ? t : (t == t ? 0.0f : t); }   // a NaN stays a NaN
// 0.5 t (1 + erf(t / sqrt 2)) with erf(x) = 1 - (a1 s + ... + a5 s^5) exp(-x^2), s = 1 / (1 + p x), x >= 0 (Abramowitz &
// Stegun 7.1.26; in FP32 arithmetic |error of erf| < 7e-7).  1 + erf is formed without cancellation on either side:
// the result is within 2e-6 relative for t >= 0 and within 1e-6 |t| absolute for t < 0.
__device__ __forceinline__ float gelu_erf(float t) {
    const float x = fabsf(t) * 0.70710678118654752f;
    const float s = __fdividef(1.0f, fmaf(0.3275911f, x, 1.0f));
    float p = fmaf(1.061405429f, s, -1.453152027f);
    p = fmaf(p, s, 1.421413741f);
    p = fmaf(p, s, -0.284496736f);
    p = fmaf(p, s, 0.254829592f);
    const float tail = p * s * __expf(-x * x);            // 1 - erf(|x|) = erfc(|x|)
    return 0.5f * t * (t >= 0.0f ? 2.0f - tail : tail);   // 1 + erf(x): 2 - erfc(|x|) right of zero, erfc(|x|) left of it
}
// 0.5 t (1 + tanh u) = t / (1 + exp(-2u)), u = sqrt(2/pi) (t + 0.044715 t^3); ex2.approx and an approximate
// division: same bounds, no branch, eight instructions
__device__ __forceinline__ float gelu_tanh(float t) {
    const float u2 = -1.5957691216057308f * t * fmaf(0.044715f * t, t, 1.0f);
    return __fdividef(t, 1.0f + __expf(u2));
}
__device__ __forceinline__ float activate(float t, int activation) {
    if (activation == 1) return relu(t);
    if (activation == 2) return gelu_erf(t);
    if (activation == 3) return gelu_tanh(t);
    return t;
}

__host__ __device__ __forceinline__ int out_dtype_bytes(int out_dtype) {
    return out_dtype == 0 ? 4 : out_dtype <= 2 ? 2 : 1;
}
__device__ __forceinline__ uint32_t pack16(float lo, float hi, int out_dtype) {
    if (out_dtype == 1) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&p);
    }
    const __half2 p = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}
// four floats -> four 8-bit floats (byte 0 = f0), round to nearest even, saturate to finite
__device__ __forceinline__ uint32_t pack8(float f0, float f1, float f2, float f3, int out_dtype) {
    const __nv_fp8_interpretation_t fmt = out_dtype == 3 ? __NV_E4M3 : __NV_E5M2;
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f0, f1), __NV_SATFINITE, fmt);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f2, f3), __NV_SATFINITE, fmt);
    return lo | (hi << 16);
}
__device__ __forceinline__ float load_out(const void* base, long long idx, int out_dtype) {
    if (out_dtype == 0) return static_cast<const float*>(base)[idx];
    if (out_dtype == 1) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    if (out_dtype == 2) return __half2float(static_cast<const __half*>(base)[idx]);
    const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<const __nv_fp8_storage_t*>(base)[idx],
                                                 out_dtype == 3 ? __NV_E4M3 : __NV_E5M2);
    return __half2float(__half(h));
}
__device__ __forceinline__ void store_out(void* base, long long idx, float v, int out_dtype) {
    if (out_dtype == 0) static_cast<float*>(base)[idx] = v;
    else if (out_dtype == 1) static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
    else if (out_dtype == 2) static_cast<__half*>(base)[idx] = __float2half_rn(v);
    else static_cast<__nv_fp8_storage_t*>(base)[idx] =
             __nv_cvt_float_to_fp8(v, __NV_SATFINITE, out_dtype == 3 ? __NV_E4M3 : __NV_E5M2);
}
// merges a thread's running maximum into the device word (non-negative floats order like their bit patterns)
__device__ __forceinline__ void amax_merge_warp(float* amax, float local) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, o));
    if ((threadIdx.x & 31) == 0 && local > 0.0f) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(local));
}

constexpr int kMaxPeers = 7;         // one box of 8 GPUs

// Diagnostic switches of GemmArgs::debug that alter results or record time stamps exist only in a library built
// with -DB200FP8_DIAGNOSTICS (csrc/Makefile, target `diag`); the product build compiles them out.
#ifdef B200FP8_DIAGNOSTICS
constexpr bool kDiagnostics = true;
#else
constexpr bool kDiagnostics = false;
#endif

struct GemmArgs {
    int M, N, K;
    int num_k_blocks;     // ceil(K / 128)
    int m_tiles;          // tiles along M (tile = 128 * CTAS rows)
    int n_tiles;          // tiles along N (tile = BN columns)
    int group_m;          // rasterisation: tiles are walked down `group_m` M-tiles before moving along N
    uint32_t idesc;       // UMMA instruction descriptor (dtype pair, tile shape)
    // Tail balancing (NACC == 1): when the last round of the persistent walk would keep at most half of the
    // CTAs busy, its `split_tiles` tiles are each processed as two half-width work items (columns [0, BN/2)
    // and [BN/2, BN)), so that the round takes half a tile time.  Work items with index >= full_items are halves.
    int full_items;       // number of full-width work items (= tiles - split_tiles)
    int split_tiles;      // tiles handled as two halves each (0 = off)
    uint32_t idesc_half;  // instruction descriptor for N = BN / 2
    int l2_loads;         // L2 eviction hint of the operand loads: 0 none, 1 evict_last, 2 evict_first
    int l2_stores;        // ... of the FP32 TMA stores of C: 0 none, 2 evict_first
    int tma_store;        // 1: TMA-store epilogue (needs ldc % 4 == 0 and 16-byte aligned C); 0: plain stores
    uint32_t wait_hint_ns; // suspend-time hint for long mbarrier waits (0 = plain polling)
    int debug;            // 512: leave the third k-block of every CTA's first tile unloaded (exercises the bounded waits).
                          // Diagnostics build only (results become wrong): 1 skip TMA loads, 2 skip C stores, 4 skip MMAs,
                          // 64 record per-k-block clock64 stamps of CTA 0's MMA warp in `trace`, 128 per-tile start stamps
    float* C;
    long long ldc;
    int* status;          // device status word: 0 = ok, else first error code recorded
    unsigned int* pace;   // tile-pacing counter (zero at launch) or nullptr: see the producer warp
    unsigned int pace_limit_ns;
    // Die-aware start positions (nullptr = off).  side_mask: bit s set = SM s sits at the second half of the L2;
    // tickets[0 / 1]: zero at launch.  CTAs (pairs) on the first side take start positions 0, 1, 2, ... of the
    // persistent walk, those on the second side tile_step - 1, tile_step - 2, ...: within every round of the walk
    // each die then works on its own contiguous run of tiles, i.e. on its own B panels, which cross the die-to-die
    // fabric for one die instead of two.
    unsigned int* tickets;
    unsigned long long side_mask[3];
    unsigned int store_gap_ns;   // pause between an epilogue warp's chunk stores (spreads C writes over the next main loop)
    long long* trace;     // diagnostics (debug & 64): per k-block clock64 stamps of CTA 0's MMA thread
    // Fused all-gather of C (N-sharded multi-GPU run): every finished box is also stored, with plain
    // 16-byte stores over NVLink, into the same position of the C matrix of each peer GPU.
    // peer_c[p] points at this rank's column block inside peer p's full matrix (row pitch ldc).
    // Blocked-ELL sparse A (CTAS == 1 only; block = 128 rows x 128 columns = one M-tile x one k-block): tmap_a
    // describes the compact values matrix [M][num_k_blocks * 128], and k-block kb of M-tile mt multiplies the
    // columns [col * 128, col * 128 + 128) of B with col = ell_col_ind[mt * num_k_blocks + kb]; col < 0 is a
    // padding block that contributes nothing (both operands are then loaded from outside the matrices: zeros).
    const int* ell_col_ind;
    int ell_oob_a, ell_oob_b;     // 128-aligned k coordinates beyond the compact A / beyond B's K
    Epilogue epi;
    int num_peers;
    float* peer_c[kMaxPeers];
    // Same, through NVSwitch multicast: one multimem store per 16 bytes reaches every GPU's matrix (own included),
    // so each box crosses this GPU's NVLink once instead of once per peer.  Replaces the TMA store and peer_c.
    float* mc_c;
};

enum : int {
    kStatusOk = 0,
    kStatusProducerTimeout = 101,
    kStatusMmaTimeout = 102,
    kStatusEpilogueTimeout = 103,
    kStatusSkinnyTimeout = 104,
};

constexpr int kBlockK = 128;         // bytes (= FP8 elements) of K per ring slot: one swizzle-128B row
constexpr int kTileM = 128;          // accumulator rows per CTA = TMEM lanes
constexpr int kEpiWarps = 8;          // two groups of four (one warp per TMEM lane quarter in each group)
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait on an mbarrier phase.  A few immediate tests first (the common case: the phase
// is already complete or completes within the round trip), then tests that let the hardware
// suspend the thread for up to `hint_ns` at a time, which keeps waiting warps from burning
// issue slots and power.  Gives up after kWaitLimitNs or when the CTA's abort flag is raised.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             bool cluster_scope, uint32_t hint_ns = 0) {
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
        const bool ok = cluster_scope ? ptx::mbar_try_wait_cluster(bar, parity) : ptx::mbar_try_wait(bar, parity);
        if (ok) return true;
    }
    uint32_t spins = 0;
    uint64_t t0 = 0;
    const uint32_t check_mask = hint_ns ? 0x7u : 0x3FFu;
    for (;;) {
        bool ok;
        if (hint_ns)
            ok = cluster_scope ? ptx::mbar_try_wait_cluster_hint(bar, parity, hint_ns) : ptx::mbar_try_wait_hint(bar, parity, hint_ns);
        else
            ok = cluster_scope ? ptx::mbar_try_wait_cluster(bar, parity) : ptx::mbar_try_wait(bar, parity);
        if (ok) return true;
        if ((++spins & check_mask) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = ptx::globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) return false;
        }
    }
}

__device__ __forceinline__ void record_failure(int* status, volatile int* abort_flag, int code) {
    *abort_flag = 1;
    if (status) atomicCAS(status, 0, code);
    __threadfence_block();
}

// STAGES ring stages of KPS k-blocks each: a stage is loaded, awaited, consumed and released as a whole (one full and
// one empty barrier per stage), so "2-stage" (gemm::GEMM) means two stages in flight, each as many k-blocks as fit.
// AROWS < 128 (one-CTA kernels, problems of at most AROWS rows): the A box holds only AROWS rows, so a slot shrinks to
// AROWS + BN rows and the ring holds more k-blocks of B in flight (decode-shaped problems stream B from HBM).  The MMA
// still reads 128 rows from the slot's start; what lies behind the box feeds accumulator rows that are never stored.
template <int BN, int STAGES, int CTAS, int NACC, int KPS = 1, int AROWS = kTileM>
struct GemmSmem {
    static constexpr int kSlots = STAGES * KPS;              // k-block slots in the ring
    static constexpr int kABytes = AROWS * kBlockK;
    static constexpr int kBRows = BN / CTAS;                 // rows of one B sub-tile held by this CTA
    static constexpr int kBBytes = kBRows * kBlockK;
    static constexpr int kStageBytes = kABytes + NACC * kBBytes;   // bytes of one k-block slot
    static constexpr int kTxBytes = kStageBytes * CTAS;      // bytes landing per k-block slot across the pair
    static constexpr int kEpiBufBytes = 32 * 32 * 4;         // one 32x32 FP32 box
    static constexpr int kEpiBytes = kEpiWarps * kEpiBufBytes;   // one staging box per epilogue warp
    static constexpr int kRingOff = 0;
    static constexpr int kEpiOff = kSlots * kStageBytes;
    static constexpr int kBarOff = kEpiOff + kEpiBytes;      // full[STAGES] empty[STAGES] tfull[2] tempty[2]
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemSlotOff = kBarOff + 8 * kNumBars;
    static constexpr int kAbortOff = kTmemSlotOff + 8;
    static constexpr int kTotal = kAbortOff + 8;
    static constexpr int kDynamicBytes = kTotal + 1024;      // slack for manual 1024-byte alignment
    static constexpr int kTmemCols = 2 * BN;                 // two accumulator slots (256 or 512 columns: powers of 2)
    static constexpr int kTileN = BN * NACC;                 // columns of C per tile
};

template <int BN, int STAGES, int CTAS, int NACC, int KPS = 1, int AROWS = kTileM>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_fp8_rowcol_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_c,
                       const __grid_constant__ CUtensorMap tmap_b_half,   // B with boxes of half as many rows (tail items)
                       const GemmArgs args)
{
    using L = GemmSmem<BN, STAGES, CTAS, NACC, KPS, AROWS>;
    static_assert(AROWS == kTileM || (CTAS == 1 && NACC == 1 && AROWS % 8 == 0), "short A boxes: one-CTA kernels only");
    static_assert(BN % 32 == 0 && BN <= 256 && (BN / CTAS) % 8 == 0 && (NACC == 1 || NACC == 2), "tile");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_addr(smem_raw));

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // provably warp-uniform
    const int lane = threadIdx.x & 31;
    const uint32_t rank = (CTAS == 2) ? ptx::cluster_ctarank() : 0u;
    const bool pair = (CTAS == 2);

    const uint32_t bar_full = smem_base + L::kBarOff;
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t tmem_slot = smem_base + L::kTmemSlotOff;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kAbortOff);
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kTmemSlotOff);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, (kEpiWarps / NACC) * CTAS);   // warps that drain one slot, in all CTAs
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        ptx::prefetch_tensormap(&tmap_c);
    }
    if (warp == 1) {
        ptx::tmem_alloc<CTAS>(tmem_slot, L::kTmemCols);
        ptx::tmem_relinquish<CTAS>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (pair) { ptx::cluster_arrive(); ptx::cluster_wait(); }
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;
    // Everything above touched only this CTA's own resources and may overlap the previous kernel's tail;
    // global memory (operands, C, pacing counter, status word) is touched only after the grids before this one are
    // complete.  The next kernel of the stream may be set up while this one runs; its own wait holds it back.
    ptx::griddep_wait();
    ptx::griddep_launch_dependents();

    // persistent walk over work items, identical in every role
    const int num_items = args.full_items + 2 * args.split_tiles;
    const int tile_step = gridDim.x / CTAS;
    int first_tile = blockIdx.x / CTAS;
    if (args.tickets != nullptr) {
        volatile int* ticket_slot = reinterpret_cast<volatile int*>(smem_gen + L::kAbortOff + 4);
        if (rank == 0 && threadIdx.x == 0) {
            const unsigned int smid = ptx::smid();
            const unsigned int side = smid < 192u ? static_cast<unsigned int>((args.side_mask[smid >> 6] >> (smid & 63u)) & 1ull) : 0u;
            const int drawn = static_cast<int>(atomicAdd(args.tickets + side, 1u));
            const int pos = side ? tile_step - 1 - drawn : drawn;
            *ticket_slot = (pos >= 0 && pos < tile_step) ? pos : first_tile;
        }
        __syncwarp();
        if (pair) {
            ptx::cluster_arrive();                        // release / acquire: the leader's slot is visible to its peer
            ptx::cluster_wait();
            first_tile = rank == 0 ? *ticket_slot : static_cast<int>(ptx::ld_shared_cluster_u32(ptx::mapa(smem_base + L::kAbortOff + 4, 0)));
        } else {
            __syncthreads();
            first_tile = *ticket_slot;
        }
    }
    const int nkb = args.num_k_blocks;
    // k-blocks this CTA streams over all of its work items: the last stage of the stream may hold fewer than KPS
    const long long stream_kb = first_tile < num_items
        ? static_cast<long long>((num_items - first_tile + tile_step - 1) / tile_step) * nkb : 0;

    // work item -> first row / column of this CTA's part; `half` = half-width tail item
    auto tile_coords = [&](int t, int& m0, int& n0, bool& half) {
        half = t >= args.full_items;
        int tile = t, h = 0;
        if (half) {
            const int u = t - args.full_items;
            tile = args.full_items + (u >> 1);
            h = u & 1;
        }
        const int per_group = args.group_m * args.n_tiles;
        const int g = tile / per_group;
        const int first_m = g * args.group_m;
        const int gsz = min(args.group_m, args.m_tiles - first_m);
        const int r = tile - g * per_group;
        const int m_blk = first_m + r % gsz;
        const int n_blk = r / gsz;
        m0 = m_blk * (kTileM * CTAS) + static_cast<int>(rank) * kTileM;
        n0 = n_blk * L::kTileN + h * (BN / 2);
    };
    // Accumulator slot bookkeeping.  NACC == 1: tile `it` owns slot it & 1 (its (it >> 1)-th use).
    // NACC == 2: every tile owns both slots (slot j holds columns [j*BN, (j+1)*BN); use number = it).
    auto slot_of = [&](int it, int j) { return NACC == 1 ? (it & 1) : j; };
    auto use_parity = [&](int it) { return static_cast<uint32_t>((NACC == 1 ? (it >> 1) : it) & 1); };

    if (warp == 0) {
        // ---------------- TMA producer: warp-uniform loop, one elected lane issues ----------------
        const uint32_t full0 = pair ? ptx::mapa(bar_full, 0) : bar_full;   // the leader's full barriers
        const uint64_t load_policy = ptx::l2_policy(args.l2_loads);
        int s = 0;                       // k-block slot; its stage is s / KPS
        uint32_t ph = 0;
        int issued = 0;
        long long streamed = 0;
        bool ok = true;
        int it = 0;
        for (int t = first_tile; t < num_items && ok; t += tile_step, ++it) {
            int m0, n0;
            bool half;
            tile_coords(t, m0, n0, half);
            const int nb0 = n0 + static_cast<int>(rank) * (half ? L::kBRows / 2 : L::kBRows);
            const CUtensorMap* tmb = half ? &tmap_b_half : &tmap_b;
            const uint32_t tx_bytes = half ? (L::kABytes + L::kBBytes / 2) * CTAS : L::kTxBytes;
            if (args.pace != nullptr && rank == 0 && it > 0) {
                // Tile pacing: CTAs that share operand panels through L2 only profit while they sweep K
                // together, and small systematic speed differences between SMs pull them apart over a
                // long run.  Before a new tile every leader announces itself and waits -- briefly and
                // never longer than pace_limit_ns -- for the others.  Purely a performance hint: running
                // out of patience just means starting the tile unaligned.
                const unsigned int target = static_cast<unsigned int>(it) * static_cast<unsigned int>(tile_step);
                if (ptx::elect_one()) atomicAdd(args.pace, 1u);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (*reinterpret_cast<volatile unsigned int*>(args.pace) < target &&
                       ptx::globaltimer_ns() - t0 < args.pace_limit_ns)
                    __nanosleep(256);
                __syncwarp();
            }
            // blocked-ELL A: lane l holds the column block of k-block (chunk base + l); the next 32 are prefetched
            const int* ell_row = nullptr;
            int ell_cur = -1, ell_nxt = -1;
            if (CTAS == 1 && args.ell_col_ind != nullptr) {
                ell_row = args.ell_col_ind + static_cast<long long>(m0 / kTileM) * nkb;
                if (lane < nkb) ell_nxt = ell_row[lane];
            }
            for (int kb = 0; kb < nkb; ++kb) {
                const int stage = s / KPS;
                const bool stage_first = (s % KPS) == 0;
                const bool stage_last = (s % KPS) == KPS - 1 || streamed + 1 == stream_kb;
                if (stage_first && !wait_bounded(bar_empty + 8 * stage, ph ^ 1u, abort_flag, pair, args.wait_hint_ns)) {
                    record_failure(args.status, abort_flag, kStatusProducerTimeout);
                    ok = false;
                    break;
                }
                int ka = kb * kBlockK, kbx = kb * kBlockK;           // k coordinates of the A and B boxes
                if (CTAS == 1 && ell_row != nullptr) {
                    if ((kb & 31) == 0) {
                        ell_cur = ell_nxt;
                        ell_nxt = (kb + 32 + lane < nkb) ? ell_row[kb + 32 + lane] : -1;
                    }
                    const int col = __shfl_sync(0xffffffffu, ell_cur, kb & 31);
                    if (col < 0 || col >= args.ell_oob_b / kBlockK) { ka = args.ell_oob_a; kbx = args.ell_oob_b; }
                    else kbx = col * kBlockK;
                }
                const uint32_t a_dst = smem_base + L::kRingOff + s * L::kStageBytes;
                const uint32_t b_dst = a_dst + L::kABytes;
                if (KPS == 1 && (args.debug & 512) && it == 0 && kb == 2) {
                    // failure-path test: this ring slot is never armed nor loaded, so the MMA warp's bounded wait on
                    // it must run out and the kernel must end by itself with a status code
                } else if (ptx::elect_one()) {
                    const uint32_t fullb = bar_full + 8 * stage;           // this CTA's barrier of the stage
                    const uint32_t fullr = full0 + 8 * stage;              // the leader's, where the copies signal
                    if (kDiagnostics && (args.debug & 1)) {
                        if (rank == 0 && stage_last) ptx::mbar_arrive(fullb);
                    } else {
                        // the stage's byte count grows k-block by k-block; the single arrival that can close the phase
                        // comes with the stage's last k-block
                        if (rank == 0) {
                            if (stage_last) ptx::mbar_arrive_expect_tx(fullb, tx_bytes);
                            else ptx::mbar_expect_tx(fullb, tx_bytes);
                        }
                        if (pair) {
                            if (args.l2_loads) {
                                ptx::tma_load_2d_pair_hint(a_dst, &tmap_a, ka, m0, fullr, load_policy);
#pragma unroll
                                for (int j = 0; j < NACC; ++j)
                                    ptx::tma_load_2d_pair_hint(b_dst + j * L::kBBytes, tmb, kbx, nb0 + j * BN, fullr, load_policy);
                            } else {
                                ptx::tma_load_2d_pair(a_dst, &tmap_a, ka, m0, fullr);
#pragma unroll
                                for (int j = 0; j < NACC; ++j)
                                    ptx::tma_load_2d_pair(b_dst + j * L::kBBytes, tmb, kbx, nb0 + j * BN, fullr);
                            }
                        } else {
                            if (args.l2_loads) {
                                ptx::tma_load_2d_hint(a_dst, &tmap_a, ka, m0, fullb, load_policy);
#pragma unroll
                                for (int j = 0; j < NACC; ++j)
                                    ptx::tma_load_2d_hint(b_dst + j * L::kBBytes, tmb, kbx, nb0 + j * BN, fullb, load_policy);
                            } else {
                                ptx::tma_load_2d(a_dst, &tmap_a, ka, m0, fullb);
#pragma unroll
                                for (int j = 0; j < NACC; ++j)
                                    ptx::tma_load_2d(b_dst + j * L::kBBytes, tmb, kbx, nb0 + j * BN, fullb);
                            }
                        }
                    }
                }
                __syncwarp();
                ++issued;
                ++streamed;
                if (++s == L::kSlots) { s = 0; ph ^= 1u; }
            }
        }
        if (args.pace != nullptr && rank == 0) {
            // announce the iterations this pair does not have, so that nobody waits for it
            const int max_it = (num_items + tile_step - 1) / tile_step;
            if (it < max_it && ptx::elect_one()) atomicAdd(args.pace, static_cast<unsigned int>(max_it - it));
            __syncwarp();
        }
        if (!ok && rank == 0) {
            // leave no copy in flight into this CTA's shared memory: close a stage that was left half armed, then wait
            // (bounded) for the stages armed last
            if ((s % KPS) != 0 && ptx::elect_one()) ptx::mbar_arrive(bar_full + 8 * (s / KPS));
            __syncwarp();
            const int pending = issued < L::kSlots ? issued : L::kSlots;
            for (int i = 0; i < pending; ++i) {
                if (s == 0) { s = L::kSlots; ph ^= 1u; }
                --s;
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(bar_full + 8 * (s / KPS), ph) && ptx::globaltimer_ns() - t0 < kWaitLimitNs) {}
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: leader CTA, warp-uniform loop, one elected lane issues ----------------
        if (rank == 0) {
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            long long streamed = 0;
            bool ok = true;
            for (int t = first_tile; t < num_items && ok; t += tile_step, ++it) {
                const uint32_t idesc = (t >= args.full_items) ? args.idesc_half : args.idesc;
                // slot 0 of this tile must have been drained; slot 1 (NACC == 2) is awaited just before its first MMA
                if (!wait_bounded(bar_tempty + 8 * slot_of(it, 0), use_parity(it) ^ 1u, abort_flag, pair, args.wait_hint_ns)) {
                    record_failure(args.status, abort_flag, kStatusMmaTimeout);
                    break;
                }
                ptx::tc_fence_after();
                if (kDiagnostics && (args.debug & 128) && lane == 0 && it < 128) args.trace[(blockIdx.x / CTAS) * 128 + it] = static_cast<long long>(ptx::globaltimer_ns());
                for (int kb = 0; kb < nkb; ++kb) {
                    long long tr0 = 0, tr1 = 0;
                    if (kDiagnostics && (args.debug & 64) && blockIdx.x == 0) tr0 = clock64();
                    const int stage = s / KPS;
                    const bool stage_last = (s % KPS) == KPS - 1 || streamed + 1 == stream_kb;
                    if ((s % KPS) == 0 && !wait_bounded(bar_full + 8 * stage, ph, abort_flag, pair, args.wait_hint_ns)) {
                        record_failure(args.status, abort_flag, kStatusMmaTimeout);
                        ok = false;
                        break;
                    }
                    if (kDiagnostics && (args.debug & 64) && blockIdx.x == 0) tr1 = clock64();
                    ptx::tc_fence_after();
                    const uint32_t a_src = smem_base + L::kRingOff + s * L::kStageBytes;
                    const uint64_t adesc = ptx::umma_desc_k128(a_src);
#pragma unroll
                    for (int j = 0; j < NACC; ++j) {
                        if (NACC == 2 && j == 1 && kb == 0) {
                            if (!wait_bounded(bar_tempty + 8, use_parity(it) ^ 1u, abort_flag, pair, args.wait_hint_ns)) {
                                record_failure(args.status, abort_flag, kStatusMmaTimeout);
                                ok = false;
                                break;
                            }
                            ptx::tc_fence_after();
                        }
                        const uint32_t d_tmem = tmem_base + slot_of(it, j) * BN;
                        const uint64_t bdesc = ptx::umma_desc_k128(a_src + L::kABytes + j * L::kBBytes);
                        if (ptx::elect_one()) {
#pragma unroll
                            for (int k = 0; k < kBlockK / 32; ++k)   // 32 bytes of K per instruction: +2 in 16-byte units
                                if (!(kDiagnostics && (args.debug & 4))) ptx::umma_f8<CTAS>(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
                        }
                        __syncwarp();
                    }
                    if (!ok) break;
                    if (stage_last && ptx::elect_one()) {                 // the whole stage has been read: hand it back
                        if (pair) ptx::umma_commit_pair(bar_empty + 8 * stage, 0x3);
                        else ptx::umma_commit(bar_empty + 8 * stage);
                    }
                    __syncwarp();
                    ++streamed;
                    if (kDiagnostics && (args.debug & 64) && blockIdx.x == 0 && lane == 0) {
                        const int idx = it * nkb + kb;
                        if (idx < 4096) { args.trace[3 * idx] = tr0; args.trace[3 * idx + 1] = tr1; args.trace[3 * idx + 2] = clock64(); }
                    }
                    if (++s == L::kSlots) { s = 0; ph ^= 1u; }
                }
                if (ok && ptx::elect_one()) {
#pragma unroll
                    for (int j = 0; j < NACC; ++j) {
                        if (pair) ptx::umma_commit_pair(bar_tfull + 8 * slot_of(it, j), 0x3);
                        else ptx::umma_commit(bar_tfull + 8 * slot_of(it, j));
                    }
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int q = warp & 3;                                   // TMEM lane quarter this warp may read
        const int grp = (warp - 2) >> 2;                          // 0 or 1
        const uint32_t sb = smem_base + L::kEpiOff + (warp - 2) * L::kEpiBufBytes;   // this warp's staging box
        const uint32_t tempty0 = pair ? ptx::mapa(bar_tempty, 0) : bar_tempty;
        const bool issuer = ptx::elect_one();                    // this lane owns the warp's bulk-store groups
        const uint64_t store_policy = ptx::l2_policy(args.l2_stores);
        constexpr int kChunks = BN / 32 / (NACC == 1 ? 2 : 1);    // 32-column chunks this warp drains per tile
        float epi_alpha0 = 1.0f, epi_dscale = 1.0f, epi_amax = 0.0f;
        if (args.epi.active) {
            epi_alpha0 = args.epi.alpha;
            if (args.epi.a_scale) epi_alpha0 *= *args.epi.a_scale;
            if (args.epi.b_scale) epi_alpha0 *= *args.epi.b_scale;
            if (args.epi.d_scale) epi_dscale = *args.epi.d_scale;
        }
        int it = 0;
        for (int t = first_tile; t < num_items; t += tile_step, ++it) {
            int m0, n0;
            bool half;
            tile_coords(t, m0, n0, half);
            const int row0 = m0 + q * 32;
            const int chunks = half ? kChunks / 2 : kChunks;     // half-width items have half the columns (NACC == 1 only)
            const int slot = slot_of(it, grp);                    // NACC == 1: both groups share the tile's slot
            const int c_first = (NACC == 1) ? grp * chunks : 0;
            if (!wait_bounded(bar_tfull + 8 * slot, use_parity(it), abort_flag, pair, args.wait_hint_ns)) {
                record_failure(args.status, abort_flag, kStatusEpilogueTimeout);
                break;
            }
            __syncwarp();
            ptx::tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + slot * BN + c_first * 32;
            const int col_base = n0 + (NACC == 2 ? grp * BN : 0) + c_first * 32;

            // diagnostics build: time stamps along the epilogue chain of one warp (CTA 0, last item)
            long long* etrace = (kDiagnostics && (args.debug & 4096) && args.trace && blockIdx.x == 0 && warp == 2 && lane == 0 &&
                                 t + tile_step >= num_items) ? args.trace : nullptr;
            int estamp = 0;
            auto stamp = [&]() { if (etrace && estamp < 30) etrace[estamp++] = static_cast<long long>(ptx::globaltimer_ns()); };
            // extended epilogue, in registers: t = alpha' * acc + beta * old D + bias (old D read row by row),
            // running |t| maximum over the valid part, then the output scale
            auto scale = [&](uint32_t (&v)[32], int c) {
                if (!args.epi.active) return;
                const int col0 = col_base + c * 32;
                const int row = row0 + lane;
                // per-column vectors: lane l fetches element col0 + l once (one coalesced load per warp and chunk), the
                // values then travel by shuffle; columns beyond N get factor 1 / bias 0 and are never stored
                if (args.epi.b_row_scale != nullptr) {
                    const float mine = (col0 + lane < args.N) ? __ldg(args.epi.b_row_scale + col0 + lane) : 1.0f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__shfl_sync(0xffffffffu, mine, i) * __uint_as_float(v[i]));
                }
                const float epi_alpha = (args.epi.a_row_scale != nullptr && row < args.M) ? epi_alpha0 * __ldg(args.epi.a_row_scale + row) : epi_alpha0;
                if (args.epi.beta != 0.0f && row < args.M) {
                    const long long base = static_cast<long long>(row) * args.ldc + col0;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float old = (col0 + i < args.N) ? load_out(args.C, base + i, args.epi.out_dtype) : 0.0f;
                        v[i] = __float_as_uint(epi_alpha * __uint_as_float(v[i]) + args.epi.beta * old);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(epi_alpha * __uint_as_float(v[i]));
                }
                if (args.epi.bias != nullptr) {
                    const float mine = (col0 + lane < args.N) ? load_out(args.epi.bias, col0 + lane, args.epi.bias_dtype) : 0.0f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __shfl_sync(0xffffffffu, mine, i));
                }
                if (args.epi.activation == 1) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(relu(__uint_as_float(v[i])));
                } else if (args.epi.activation == 2) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(gelu_erf(__uint_as_float(v[i])));
                } else if (args.epi.activation == 3) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(gelu_tanh(__uint_as_float(v[i])));
                }
                if (args.epi.amax != nullptr && row < args.M) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < args.N) epi_amax = fmaxf(epi_amax, fabsf(__uint_as_float(v[i])));
                }
                if (args.epi.d_scale != nullptr) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(epi_dscale * __uint_as_float(v[i]));
                }
            };
            // one chunk: registers -> swizzled staging box -> TMA store (or plain stores when C is not TMA-able)
            auto emit = [&](const uint32_t (&v)[32], int c) {
                const int col0 = col_base + c * 32;
                if (args.tma_store && args.epi.out_dtype >= 3) {
                    // 8-bit output: the box is 32 rows x 32 bytes, unswizzled
                    if (issuer) ptx::bulk_wait_group_read<0>();
                    __syncwarp();
                    const uint32_t row_addr = sb + lane * 32;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            w[j] = pack8(__uint_as_float(v[16 * i + 4 * j]), __uint_as_float(v[16 * i + 4 * j + 1]),
                                         __uint_as_float(v[16 * i + 4 * j + 2]), __uint_as_float(v[16 * i + 4 * j + 3]),
                                         args.epi.out_dtype);
                        ptx::st_shared_v4(row_addr + i * 16, w[0], w[1], w[2], w[3]);
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (issuer) {
                        if (row0 < args.M && col0 < args.N) ptx::tma_store_2d(&tmap_c, sb, col0, row0);
                        ptx::bulk_commit_group();
                    }
                } else if (args.tma_store && args.epi.out_dtype != 0) {
                    // 16-bit output: the box is 32 rows x 64 bytes, unswizzled
                    if (issuer) ptx::bulk_wait_group_read<0>();
                    __syncwarp();
                    const uint32_t row_addr = sb + lane * 64;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        ptx::st_shared_v4(row_addr + i * 16, pack16(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1]), args.epi.out_dtype),
                                          pack16(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]), args.epi.out_dtype),
                                          pack16(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]), args.epi.out_dtype),
                                          pack16(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]), args.epi.out_dtype));
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (issuer) {
                        if (row0 < args.M && col0 < args.N) ptx::tma_store_2d(&tmap_c, sb, col0, row0);
                        ptx::bulk_commit_group();
                    }
                } else if (args.tma_store) {
                    if (issuer) ptx::bulk_wait_group_read<0>();   // the previous store has finished reading the box
                    __syncwarp();
                    stamp();                                      // box free
                    const uint32_t row_addr = sb + lane * 128;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        ptx::st_shared_v4(row_addr + ((i ^ (lane & 7)) << 4), v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    stamp();                                      // staged
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    stamp();                                      // fenced
                    if (issuer) {
                        if (row0 < args.M && col0 < args.N && !(kDiagnostics && (args.debug & 2)) && args.mc_c == nullptr) {
                            if (args.l2_stores) ptx::tma_store_2d_hint(&tmap_c, sb, col0, row0, store_policy);
                            else ptx::tma_store_2d(&tmap_c, sb, col0, row0);
                        }
                        ptx::bulk_commit_group();
                    }
                    if (args.num_peers > 0 || args.mc_c != nullptr) {
                        // Read the box back row-contiguously (8 lanes cover one 128-byte row, 4 rows per
                        // instruction) and push it to every peer: full 128-byte lines over NVLink.
                        uint4 w[8];
                        const int chunk = lane & 7;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = i * 4 + (lane >> 3);
                            w[i] = ptx::ld_shared_v4(sb + r * 128 + ((chunk ^ (r & 7)) << 4));
                        }
                        const int col = col0 + chunk * 4;
                        if (col < args.N && args.mc_c != nullptr) {
                            float* base = args.mc_c + col;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int row = row0 + i * 4 + (lane >> 3);
                                if (row < args.M) ptx::multimem_st_v4(base + static_cast<long long>(row) * args.ldc, w[i]);
                            }
                        } else if (col < args.N) {                 // N % 4 == 0 on this path: whole 16-byte groups
                            for (int p = 0; p < args.num_peers; ++p) {
                                float* base = args.peer_c[p] + col;
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const int row = row0 + i * 4 + (lane >> 3);
                                    if (row < args.M)
                                        *reinterpret_cast<uint4*>(base + static_cast<long long>(row) * args.ldc) = w[i];
                                }
                            }
                        }
                    }
                } else {
                    // C cannot be written by TMA (pitch, row end or base not 16-byte aligned): transpose the chunk through
                    // the staging box so that one instruction writes 32 consecutive elements of ONE row (lane = column),
                    // instead of every lane walking along its own row (32 lines touched per instruction, 2.2 x slower
                    // for the whole GEMM at 4096 x 4096 x 4098)
                    __syncwarp();                                 // the previous chunk has been read out of the box
                    const uint32_t row_addr = sb + lane * 128;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        ptx::st_shared_v4(row_addr + ((i ^ (lane & 7)) << 4), v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    __syncwarp();
                    const int col = col0 + lane;
                    const int rows = min(32, args.M - row0);
                    if (col < args.N) {
                        long long idx = static_cast<long long>(row0) * args.ldc + col;
                        for (int r = 0; r < rows; ++r, idx += args.ldc) {
                            const uint32_t w = ptx::ld_shared_u32(sb + r * 128 + ((((lane >> 2) ^ (r & 7)) << 4) | ((lane & 3) << 2)));
                            store_out(args.C, idx, __uint_as_float(w), args.epi.out_dtype);
                        }
                    }
                }
            };
            auto release_slot = [&]() {                           // accumulator columns of this warp are in registers
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (pair) ptx::mbar_arrive_cluster(tempty0 + 8 * slot);
                    else ptx::mbar_arrive(bar_tempty + 8 * slot);
                }
            };

            stamp();                                              // accumulator complete
            // two register sets: the TMEM load of chunk c+1 is in flight while chunk c is stored
            uint32_t va[32], vb[32];
            ptx::tmem_ld_32x32(t_addr, va);
            if constexpr (kChunks == 1) {                         // 64-column tile: one chunk per warp
                ptx::tmem_ld_wait();
                scale(va, 0);
                release_slot();
                emit(va, 0);
            } else
#pragma unroll 1
            for (int c = 0; c < chunks; c += 2) {
                ptx::tmem_ld_wait();                              // va = chunk c
                stamp();                                          // chunk c in registers
                ptx::tmem_ld_32x32(t_addr + (c + 1) * 32, vb);    // chunks is even: chunk c+1 exists
                scale(va, c);
                emit(va, c);
                stamp();                                          // chunk c staged, store issued
                ptx::tmem_ld_wait();                              // vb = chunk c+1
                scale(vb, c + 1);
                if (c + 2 < chunks) ptx::tmem_ld_32x32(t_addr + (c + 2) * 32, va);
                else release_slot();
                if (args.store_gap_ns) __nanosleep(args.store_gap_ns);
                emit(vb, c + 1);
                stamp();                                          // chunk c+1 staged, store issued
                if (args.store_gap_ns && c + 2 < chunks) __nanosleep(args.store_gap_ns);
            }
            if (etrace) {
                if (issuer) ptx::bulk_wait_group_read<0>();
                stamp();                                          // last store has read its box
                if (issuer) ptx::bulk_wait_group<0>();
                stamp();                                          // all of this warp's stores are complete
            }
        }
        // the staging box must outlive the stores' reads of it; the writes themselves complete with the grid
        if (issuer) ptx::bulk_wait_group_read<0>();
        __syncwarp();
        if (args.epi.amax != nullptr) amax_merge_warp(args.epi.amax, epi_amax);
    }

    // ---------------- teardown ----------------
    ptx::tc_fence_before();
    __syncthreads();
    if (pair) { ptx::cluster_arrive(); ptx::cluster_wait(); }
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc<CTAS>(tmem_base, L::kTmemCols);
    }
}

}  // namespace b200fp8
