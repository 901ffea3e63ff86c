// Host side of the C ABI declared in include/b200fp8.h: argument validation, TMA
// descriptor encoding, kernel selection and launch.  Replaces the reference's host
// launchers GEMMex / GEMMex4 (GEMM/src/gemm.cu:263-277, :670-686).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <mutex>

#include "../../include/b200fp8.h"
#include "gemm_sm100.cuh"
#include "gemm_skinny_sm100.cuh"
#include "gemm_skinny_streamk_sm100.cuh"
#include "fill_fp8.cuh"
#include "l2_sides.cuh"

namespace b200fp8 {
namespace {

constexpr int kMaxDevices = 64;
constexpr int kPaceSlots = 256;
constexpr int kPaceWords = 4;

struct DeviceCtx {
    bool ready = false;
    int sm_count = 0;
    int* status = nullptr;          // device status word
    unsigned int* pace = nullptr;   // ring of launch scratch slots, one per launch in flight: kPaceWords zeroed words
                                    // (word 0 the tile-pacing counter, words 1 and 2 the start-position tickets)
    unsigned int pace_next = 0;
    bool sides_known = false;       // side_mask holds a measured split of the SMs over the two halves of the L2
    uint64_t side_mask[3] = {0, 0, 0};
    // buffers of the host-pointer entry point
    void* host_a = nullptr; size_t host_a_bytes = 0;
    void* host_b = nullptr; size_t host_b_bytes = 0;
    void* host_c = nullptr; size_t host_c_bytes = 0;
    cudaStream_t copy_in = nullptr, compute = nullptr, copy_out = nullptr;
    std::mutex host_mutex;          // serialises the host-pointer entry point on this device (it owns the buffers above)
    StreamKWorkspace streamk;       // scratch of the stream-K split kernel, allocated at its first launch
};

std::mutex g_mutex;
DeviceCtx g_ctx[kMaxDevices];
thread_local long long t_launches = 0;

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;

cudaError_t load_encode() {
    if (g_encode) return cudaSuccess;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess) return e;
    if (q != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
    g_encode = reinterpret_cast<EncodeFn>(fn);
    return cudaSuccess;
}

cudaError_t get_ctx(DeviceCtx** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceCtx& c = g_ctx[dev];
    if (!c.ready) {
        int major = 0;
        if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return e;
        if (major != 10) return cudaErrorNoKernelImageForDevice;   // sm_100a only: no other path exists
        if ((e = cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
        if ((e = load_encode()) != cudaSuccess) return e;
        if ((e = cudaMalloc(&c.status, sizeof(int))) != cudaSuccess) return e;
        if ((e = cudaMemset(c.status, 0, sizeof(int))) != cudaSuccess) return e;
        if ((e = cudaMalloc(&c.pace, kPaceSlots * kPaceWords * sizeof(unsigned int))) != cudaSuccess) return e;
        const char* die_aware = getenv("B200FP8_DIE_AWARE");     // 0: schedule as if the L2 were one piece
        c.sides_known = (!die_aware || atoi(die_aware) != 0) && measure_l2_sides(c.sm_count, c.side_mask);
        (void)cudaGetLastError();   // a measurement that could not run is not an error of the caller
        c.ready = true;
    }
    *out = &c;
    return cudaSuccess;
}

// 2-D tensor map over a row-major matrix of `rows` x `cols` elements with row pitch `ld` elements.
// A descriptor is a pure function of these arguments, so each host thread keeps the last few it encoded: a caller
// that repeats a call with the same pointers (a benchmark loop, a layer called every step) skips the encoding.
cudaError_t encode_2d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t cols,
                      uint64_t rows, uint64_t ld, uint32_t box_cols, uint32_t box_rows,
                      CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    struct Key {
        const void* base; uint64_t cols, rows, ld; uint32_t box_cols, box_rows; int type, elem_bytes, swizzle;
        bool operator==(const Key& o) const {
            return base == o.base && cols == o.cols && rows == o.rows && ld == o.ld && box_cols == o.box_cols &&
                   box_rows == o.box_rows && type == o.type && elem_bytes == o.elem_bytes && swizzle == o.swizzle;
        }
    };
    constexpr int kSlots = 16;
    struct Cache { Key key[kSlots]; CUtensorMap map[kSlots]; bool used[kSlots]; };
    static thread_local Cache cache = {};
    const Key key{base, cols, rows, ld, box_cols, box_rows, static_cast<int>(type), elem_bytes, static_cast<int>(swizzle)};
    const uint64_t h = (reinterpret_cast<uintptr_t>(base) >> 8) * 0x9E3779B97F4A7C15ull + cols * 31 + rows * 131 + box_rows * 7 + box_cols;
    const int slot = static_cast<int>((h >> 32) % kSlots);
    if (cache.used[slot] && cache.key[slot] == key) { *map = cache.map[slot]; return cudaSuccess; }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    // L2 promotion of the copies: 256 bytes measured best or equal everywhere (B200FP8_L2_PROMOTION=0..3: none/64/128/256)
    static const CUtensorMapL2promotion promo = [] {
        const char* v = getenv("B200FP8_L2_PROMOTION");
        const int p = v ? atoi(v) : 3;
        return p == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : p == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
             : p == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    }();
    CUresult r = g_encode(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    cache.key[slot] = key; cache.map[slot] = *map; cache.used[slot] = true;
    return cudaSuccess;
}

// Destinations of the fused all-gather epilogue: this rank's column block inside every peer's C.
struct PeerSet {
    int count = 0;
    float* c[kMaxPeers] = {};
    float* multicast = nullptr;      // when set, one multimem store replaces the own store and all peer stores
};

// Tuning knobs read once from the environment (B200FP8_*); defaults are the measured best.
struct Tune {
    int wait_hint_ns = 0;
    int group_m_pair = 16;
    int group_m_single = 16;
    int debug = 0;
    int pace_min_waves = 8;       // tile pacing only pays on long runs
    int pace_limit_ns = 30000;
    int store_gap_ns = 0;
    int split_tail = 1;
    int l2_loads = 0, l2_stores = 0;   // L2 eviction hints of operand loads / C stores (see GemmArgs)
    int pdl = 1;                  // launch with programmatic stream serialization (set-up overlaps the previous kernel's tail)
    int host_block_m = 4096;      // host-pointer entry: edge of the C blocks it pipelines over (rows / columns)
    int host_block_n = 4096;
    Tune() {
        if (const char* v = getenv("B200FP8_PDL")) pdl = atoi(v);
        if (const char* v = getenv("B200FP8_L2_LOADS")) l2_loads = atoi(v);
        if (const char* v = getenv("B200FP8_L2_STORES")) l2_stores = atoi(v);
        if (const char* v = getenv("B200FP8_HOST_BLOCK_M")) host_block_m = atoi(v) >= 256 ? atoi(v) : host_block_m;
        if (const char* v = getenv("B200FP8_HOST_BLOCK_N")) host_block_n = atoi(v) >= 256 ? atoi(v) : host_block_n;
        if (const char* v = getenv("B200FP8_SPLIT_TAIL")) split_tail = atoi(v);
        if (const char* v = getenv("B200FP8_STORE_GAP_NS")) store_gap_ns = atoi(v);
        if (const char* v = getenv("B200FP8_PACE_MIN_WAVES")) pace_min_waves = atoi(v);
        if (const char* v = getenv("B200FP8_PACE_LIMIT_NS")) pace_limit_ns = atoi(v);
        if (const char* v = getenv("B200FP8_DEBUG")) debug = atoi(v);
        if (const char* v = getenv("B200FP8_WAIT_HINT_NS")) wait_hint_ns = atoi(v);
        if (const char* v = getenv("B200FP8_GROUP_M_PAIR")) group_m_pair = atoi(v) > 0 ? atoi(v) : group_m_pair;
        if (const char* v = getenv("B200FP8_GROUP_M_SINGLE")) group_m_single = atoi(v) > 0 ? atoi(v) : group_m_single;
    }
};
const Tune& tune() { static Tune t; return t; }
#ifdef B200FP8_DIAGNOSTICS
long long* g_trace = nullptr;   // time-stamp buffer of the diagnostics build (B200FP8_DEBUG & (64 | 128 | 1024))
constexpr int kTraceWords = 3 * 4096;
long long* trace_buffer() {
    if (!g_trace && cudaMalloc(&g_trace, kTraceWords * sizeof(long long)) == cudaSuccess)
        cudaMemset(g_trace, 0, kTraceWords * sizeof(long long));
    return g_trace;
}
#endif

// One workspace slot of the stream-K kernel for the next launch (allocated on first use: four slots of one parked
// tile and one flag per SM).
cudaError_t streamk_slot(DeviceCtx& ctx, float4** scratch, unsigned int** flags) {
    std::lock_guard<std::mutex> lock(g_mutex);
    StreamKWorkspace& w = ctx.streamk;
    if (w.max_ctas == 0) {
        for (int i = 0; i < StreamKWorkspace::kSlots; ++i) {
            cudaError_t e = cudaMalloc(&w.scratch[i], StreamKWorkspace::scratch_bytes(ctx.sm_count));
            if (e == cudaSuccess) e = cudaMalloc(&w.flags[i], ctx.sm_count * sizeof(unsigned int));
            if (e == cudaSuccess) e = cudaMemset(w.flags[i], 0, ctx.sm_count * sizeof(unsigned int));
            if (e != cudaSuccess) return e;
        }
        w.max_ctas = ctx.sm_count;
    }
    const unsigned int i = w.next++ % StreamKWorkspace::kSlots;
    *scratch = w.scratch[i];
    *flags = w.flags[i];
    return cudaSuccess;
}

// Blocked-ELL description of A (128 x 128 blocks): column-block indices [ceil(M/128)][blocks] on the device
struct EllSpec {
    const int* col_ind;
    int blocks;
};

template <int BN, int STAGES, int CTAS, int NACC, int KPS = 1, int AROWS = kTileM>
cudaError_t launch_main(DeviceCtx& ctx, int m, int k, int n, const void* a, long long lda, const void* b,
                        long long ldb, float* c, long long ldc, int a_dtype, int b_dtype, int max_ctas,
                        const PeerSet* peers, const Epilogue* epi, cudaStream_t stream, const EllSpec* ell = nullptr) {
    using L = GemmSmem<BN, STAGES, CTAS, NACC, KPS, AROWS>;
    static bool attr_done[kMaxDevices] = {};
    if (AROWS < kTileM && (m > AROWS || ell)) return cudaErrorInvalidValue;   // the short A box holds the whole M
    if (ell && CTAS != 1) return cudaErrorInvalidValue;       // a block row is one 128-row M-tile
    auto kernel = gemm_fp8_rowcol_kernel<BN, STAGES, CTAS, NACC, KPS, AROWS>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    GemmArgs args{};
    args.M = m; args.N = n; args.K = k;
    args.num_k_blocks = ell ? ell->blocks : (k + kBlockK - 1) / kBlockK;
    if (ell) {
        args.ell_col_ind = ell->col_ind;
        args.ell_oob_a = ell->blocks * kBlockK;
        args.ell_oob_b = (k + kBlockK - 1) / kBlockK * kBlockK;
    }
    args.m_tiles = (m + kTileM * CTAS - 1) / (kTileM * CTAS);
    args.n_tiles = (n + L::kTileN - 1) / L::kTileN;
    args.group_m = (CTAS == 2) ? tune().group_m_pair : tune().group_m_single;
    args.wait_hint_ns = static_cast<uint32_t>(tune().wait_hint_ns);
    args.l2_loads = tune().l2_loads;
    args.l2_stores = tune().l2_stores;
    args.debug = tune().debug;
    args.store_gap_ns = (NACC == 1) ? static_cast<unsigned int>(tune().store_gap_ns) : 0u;
#ifdef B200FP8_DIAGNOSTICS
    if (args.debug & (64 | 128 | 4096)) args.trace = trace_buffer();
    if (!args.trace) args.debug &= ~(64 | 128 | 4096);
#endif
    args.idesc = make_idesc_f8(a_dtype, b_dtype, kTileM * CTAS, BN);
    const int out_bytes = epi ? out_dtype_bytes(epi->out_dtype) : 4;
    // TMA stores clip at 16-byte granularity: a row end that is not a multiple of 16 bytes would spill into the
    // pitch padding, so such shapes take the plain-store epilogue
    args.tma_store = (((ldc * out_bytes) % 16) == 0 && ((static_cast<long long>(n) * out_bytes) % 16) == 0 &&
                      (reinterpret_cast<uintptr_t>(c) % 16) == 0) ? 1 : 0;
    args.C = c; args.ldc = ldc; args.status = ctx.status;
    if (epi) args.epi = *epi;
    if (epi && epi->active && peers && (peers->count > 0 || peers->multicast)) return cudaErrorInvalidValue;
    if (peers && (peers->count > 0 || peers->multicast)) {
        if (!args.tma_store || (n % 4) != 0) return cudaErrorInvalidValue;     // peer stores move whole 16-byte groups
        if (peers->multicast) {
            args.mc_c = peers->multicast;
        } else {
            args.num_peers = peers->count;
            for (int i = 0; i < peers->count; ++i) args.peer_c[i] = peers->c[i];
        }
    }

    CUtensorMap ta, tb, tc;
    cudaError_t e;
    const long long a_cols = ell ? static_cast<long long>(ell->blocks) * kBlockK : k;
    if ((e = encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, a_cols, m, lda, kBlockK, AROWS)) != cudaSuccess) return e;
    if ((e = encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, k, n, ldb, kBlockK, L::kBRows)) != cudaSuccess) return e;
    if (args.tma_store && out_bytes == 1) {
        if ((e = encode_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, c, n, m, ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_NONE)) != cudaSuccess) return e;
    } else if (args.tma_store && out_bytes == 2) {
        const CUtensorMapDataType t16 = epi->out_dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        if ((e = encode_2d(&tc, t16, 2, c, n, m, ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_NONE)) != cudaSuccess) return e;
    } else if (args.tma_store) {
        if ((e = encode_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, c, n, m, ldc, 32, 32)) != cudaSuccess) return e;
    } else {
        tc = ta;   // unused by the kernel on this path; any valid descriptor
    }

    const long long tiles = static_cast<long long>(args.m_tiles) * args.n_tiles;
    if (tiles > (1LL << 30)) return cudaErrorInvalidValue;
    int units = ctx.sm_count / CTAS;                     // CTAs (or pairs) resident at once
    if (max_ctas > 0 && max_ctas / CTAS < units) units = max_ctas / CTAS > 0 ? max_ctas / CTAS : 1;
    if (tiles < units) units = static_cast<int>(tiles);
    // tail balancing: a last round that would occupy at most half of the CTAs is run as half-width items
    const int rem = static_cast<int>(tiles % units);
    const bool split_tail = NACC == 1 && BN == 256 && tune().split_tail && tiles > units && rem > 0 && 2 * rem <= units;
    args.split_tiles = split_tail ? rem : 0;
    args.full_items = static_cast<int>(tiles) - args.split_tiles;
    args.idesc_half = make_idesc_f8(a_dtype, b_dtype, kTileM * CTAS, BN / 2);
    CUtensorMap tbh = tb;
    if (split_tail &&
        (e = encode_2d(&tbh, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, k, n, ldb, kBlockK, L::kBRows / 2)) != cudaSuccess)
        return e;

    // tile pacing for long persistent runs (pairs only): a fresh zeroed counter per launch, stream-ordered
    if (CTAS == 2 && tune().pace_min_waves > 0 && tiles >= static_cast<long long>(tune().pace_min_waves) * units) {
        unsigned int* slot;
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            slot = ctx.pace + kPaceWords * (ctx.pace_next++ % kPaceSlots);
        }
        if ((e = cudaMemsetAsync(slot, 0, kPaceWords * sizeof(unsigned int), stream)) != cudaSuccess) return e;
        args.pace = slot;
        args.pace_limit_ns = static_cast<unsigned int>(tune().pace_limit_ns);
        if (ctx.sides_known && units * CTAS == ctx.sm_count) {   // every SM holds exactly one CTA: the tickets of the two sides cannot collide
            args.tickets = slot + 1;
            for (int i = 0; i < 3; ++i) args.side_mask[i] = ctx.side_mask[i];
        }
    }

    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(units * CTAS), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynamicBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see griddep_wait in the kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tune().pdl ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, tbh, args);
    if (e == cudaSuccess) ++t_launches;
    return e;
}

bool valid_dtype(int d) { return d == B200FP8_E4M3 || d == B200FP8_E5M2; }

// The automatic choice among the kernels for an M x K x N problem (sparse: blocked-ELL A).  Every rule carries the
// measurement that decided it; `planner_audit.py` checks the whole table against forced kernels.
int choose_kernel(int sm_count, int m, int k, int n, bool ell) {
    int kernel = B200FP8_KERNEL_AUTO;
    const long long pair_tiles = static_cast<long long>((m + 255) / 256) * ((n + 255) / 256);
    const long long n256_tiles = static_cast<long long>((m + 127) / 128) * ((n + 255) / 256);
    const long long wide_tiles = static_cast<long long>((m + 255) / 256) * ((n + 511) / 512);
    const long long n128_cols = (n + 127) / 128;
    if (ell) kernel = n256_tiles >= sm_count / 2 ? B200FP8_KERNEL_CTA1_N256 : B200FP8_KERNEL_CTA1_N128;
    // M <= 128: the split-K kernel streams a big B from HBM with every SM; with a short K and at most one round of
    // 128 x 64 tiles there is nothing to split and its reduce-scatter only costs (128 x 2048 x 2048: 12.7 us
    // against 6.7 us for the tile kernel), so those go to the tile kernels: K <= 2048 for M > 64, K <= 1024 for
    // 32 < M <= 64 (64 x 2048 x 4096: 5.5 us split in two against 5.9; 64 x 512 x 8192: 3.9 against 5.1 the other way),
    // K <= 512 for 16 < M <= 32 (32 x 512 x 8192: 3.7 against 4.3; but 32 x 1024 x 2048: 3.9 against 4.1 the other way),
    // never for M <= 16 (16 x 512 x 2048: 3.3 against 3.5)
    else if (m <= kSkinnyMaxM && m > 16 && k <= (m > 64 ? 2048 : m > 32 ? 1024 : 512) && (n + 63) / 64 <= sm_count)
        kernel = 2 * n128_cols <= sm_count ? B200FP8_KERNEL_CTA1_N64 : B200FP8_KERNEL_CTA1_N128;
    else if (m <= kSkinnyMaxM) kernel = B200FP8_KERNEL_SKINNY;
    // at most 128 columns: tiles of 256 columns would compute padding for half of their width
    // (16384 x 4096 x 128: 11.7 us with 128 x 128 tiles against 16.2-16.5 with the 256-wide ones)
    // one round of 256 x 128 pair tiles is level with or ahead of one round of 128 x 128 tiles (12.6 against 14.0-15.0 us on one box, 11.8 both on another)
    else if (n <= 128)
        kernel = 2 * static_cast<long long>((m + 127) / 128) <= sm_count ? B200FP8_KERNEL_CTA1_N64
                 : (m + 255) / 256 <= sm_count / 2                        ? B200FP8_KERNEL_PAIR_N128
                                                                               : B200FP8_KERNEL_CTA1_N128;
    // Long runs are power-limited and the wide tile moves a quarter less data per flop, but it has no second
    // accumulator slot, so its epilogue (about 5 us) is exposed once per tile: it pays when a tile's main loop
    // is long.  Measured against the 256 x 256 pair tile: K = 32768 wins 5-8 % from 7 rounds of tiles on
    // (32768 x 32768 x 2048..8192, 8192 x 32768 x 8192), K = 28672 5 % (8192 x 28672 x 8192; at 3.5 rounds it loses
    // 7 %), K = 24576 ties, K = 20480 loses; K = 16384 wins 3-8 % at 28 rounds (16384^3), is anywhere between
    // +3 and -10 % at 14 rounds (16384 x 16384 x 8192, either way round) and loses 4-9 % at 7-10 rounds; K = 8192 loses
    // 4-15 % everywhere (8192 x 8192 x 28672: 1580 against 1435 us).
    else if ((k >= 28672 && wide_tiles >= 4LL * (sm_count / 2)) || (k >= 16384 && wide_tiles >= 20LL * (sm_count / 2)))
        kernel = B200FP8_KERNEL_PAIR_N512;
    // a short K makes the step a store of C with some arithmetic attached: one-CTA 128 x 256 tiles drain their
    // accumulators from twice as many independent CTAs as the pairs do (4096 x 512 x 4096: 15.9 against 18.7 us,
    // 8192 x 512 x 8192: 55 against 75-78, 8192 x 1024 x 8192: 81-84 against 92-93, 2304 x 1024 x 2304: 10.5 against 12.0;
    // at K = 1536 and 2048 the pair tile leads again)
    else if (k <= 1024 && n256_tiles >= sm_count / 2) kernel = B200FP8_KERNEL_CTA1_N256;
    else if (pair_tiles >= sm_count / 2) {
        kernel = B200FP8_KERNEL_PAIR_N256;
        // few rounds: count them.  A last round of at most half the pairs costs half a round (it runs as
        // half-width items); the one-CTA tile is about a tenth slower per round but its rounds hold twice as many
        // tiles of half the height (1152 x 8192 x 4096: 80 pair tiles = 1.5 rounds, 144 one-CTA tiles = 1: 33.0 against 38.8 us)
        const long long pairs = sm_count / 2;
        if (pair_tiles < 4 * pairs) {
            const long long rem = pair_tiles % pairs;
            const double rounds_pair = static_cast<double>(pair_tiles / pairs) + (rem == 0 ? 0.0 : 2 * rem <= pairs ? 0.5 : 1.0);
            const double rounds_single = static_cast<double>((n256_tiles + sm_count - 1) / sm_count);
            if (1.1 * rounds_single < rounds_pair) kernel = B200FP8_KERNEL_CTA1_N256;
        }
    }
    // a long K with three quarters of the pairs busy: the pair tile's lower traffic per flop still wins (measured
    // at M = 300..512, N = K = 8192: 3-8 %); with a short K the one-CTA kernel's smaller tail does
    else if (4 * pair_tiles >= 3 * (sm_count / 2) && k >= 8192) kernel = B200FP8_KERNEL_PAIR_N256;
    // one row of 256 x 128 pair tiles that fills most of the pairs: a quarter less operand traffic per CTA than
    // 128 x 128 tiles (measured at M = 130..256, N = K = 8192: 5-7 %)
    else if (m <= 256 && k >= 8192 && 4 * n128_cols >= 3 * (sm_count / 2) && n128_cols <= sm_count / 2)
        kernel = B200FP8_KERNEL_PAIR_N128;
    // ... and the same for one or two columns of tiles under a tall A (8192 x 8192 x 136..256: 16.3-17.9 against 17.4-18.7 us)
    else if (n > 128 && n <= 256 && k >= 8192 && 8LL * ((m + 255) / 256) >= 3 * (sm_count / 2) && 2LL * ((m + 255) / 256) <= sm_count / 2)
        kernel = B200FP8_KERNEL_PAIR_N128;
    // one round either way: with K >= 4096 the pair's shared B (32 instead of 48 KiB per CTA and k-block) wins 2-6 %
    // (640 x 5120 x 5120, 200 x 4096 x 11008, 1024 x 4096 x 4096, 8192 x 8192 x 512); with a shorter K the one-CTA tile does
    else if (n256_tiles >= sm_count / 2)
        kernel = (k >= 4096 && 2 * pair_tiles <= sm_count) ? B200FP8_KERNEL_PAIR_N256 : B200FP8_KERNEL_CTA1_N256;
    // a problem of so few 128 x 128 tiles that twice as many 128 x 64 tiles still fit in one round: half the
    // main loop and half the epilogue per CTA (1024^3: 6.4 -> 5.5 us, 256^3: 5.2 -> 4.2 us)
    else if (2 * static_cast<long long>((m + 127) / 128) * n128_cols <= sm_count) kernel = B200FP8_KERNEL_CTA1_N64;
    else kernel = B200FP8_KERNEL_CTA1_N128;
    return kernel;
}

cudaError_t gemm_dispatch(int m, int k, int n, const void* a, int a_dtype, long long lda, const void* b, int b_dtype,
                          long long ldb, float* c, long long ldc, const b200fp8_options* opt, cudaStream_t stream,
                          const PeerSet* peers = nullptr, const Epilogue* epi = nullptr, const EllSpec* ell = nullptr) {
    if (m < 0 || n < 0 || k < 0 || !valid_dtype(a_dtype) || !valid_dtype(b_dtype)) return cudaErrorInvalidValue;
    if (ell && (ell->blocks < 0 || ell->blocks > (1 << 20) ||
                (ell->blocks > 0 && (!ell->col_ind || (reinterpret_cast<uintptr_t>(ell->col_ind) % 4)))))
        return cudaErrorInvalidValue;
    if (m == 0 || n == 0) return cudaSuccess;
    if (!c || ldc < n) return cudaErrorInvalidValue;
    if (epi && epi->active && k == 0) return cudaErrorInvalidValue;   // the extended form needs a non-empty K
    if (k == 0 || (ell && ell->blocks == 0))
        return cudaMemset2DAsync(c, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(n) * 4, m, stream);
    if (!a || !b || lda < (ell ? static_cast<long long>(ell->blocks) * kBlockK : k) || ldb < k) return cudaErrorInvalidValue;
    if ((k % 16) || (lda % 16) || (ldb % 16)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(a) % 16) || (reinterpret_cast<uintptr_t>(b) % 16) ||
        (reinterpret_cast<uintptr_t>(c) % (epi ? out_dtype_bytes(epi->out_dtype) : 4)))
        return cudaErrorInvalidValue;

    int depth = opt ? opt->depth : 0;
    int kernel = opt ? opt->kernel : B200FP8_KERNEL_AUTO;
    const int split_k = opt ? opt->split_k : 0;
    const int max_ctas = opt ? opt->max_ctas : 0;
    if (depth != 0 && depth != 2 && depth != 4) return cudaErrorInvalidValue;
    if (kernel < B200FP8_KERNEL_AUTO || kernel > B200FP8_KERNEL_SKINNY_STREAMK) return cudaErrorInvalidValue;
    if (split_k > 64) return cudaErrorInvalidValue;
    if (split_k < 0 || max_ctas < 0) return cudaErrorInvalidValue;

    DeviceCtx* ctx = nullptr;
    cudaError_t e = get_ctx(&ctx);
    if (e != cudaSuccess) return e;

    if (kernel == B200FP8_KERNEL_AUTO) kernel = choose_kernel(ctx->sm_count, m, k, n, ell != nullptr);
    if ((kernel == B200FP8_KERNEL_SKINNY || kernel == B200FP8_KERNEL_SKINNY_STREAMK) && m > kSkinnyMaxM) return cudaErrorInvalidValue;
    if (ell && kernel != B200FP8_KERNEL_CTA1_N256 && kernel != B200FP8_KERNEL_CTA1_N128 && kernel != B200FP8_KERNEL_CTA1_N64)
        return cudaErrorInvalidValue;
    if (peers && (peers->count > 0 || peers->multicast) && (kernel == B200FP8_KERNEL_SKINNY || kernel == B200FP8_KERNEL_SKINNY_STREAMK))
        kernel = B200FP8_KERNEL_PAIR_N256;

    // Ring depth: `depth` stages in flight (2 = gemm::GEMM, 4 = gemm::GEMM4), each stage as many 128-byte k-blocks as
    // shared memory holds (KPS); depth 0 = one k-block per stage, as many stages as fit.
#define B200FP8_LAUNCH5(BN, ST, CT, NA, KPS) \
    launch_main<BN, ST, CT, NA, KPS>(*ctx, m, k, n, a, lda, b, ldb, c, ldc, a_dtype, b_dtype, max_ctas, peers, epi, stream, ell)
#define B200FP8_LAUNCH6(BN, ST, CT, NA, KPS, AR) \
    launch_main<BN, ST, CT, NA, KPS, AR>(*ctx, m, k, n, a, lda, b, ldb, c, ldc, a_dtype, b_dtype, max_ctas, peers, epi, stream, ell)
    switch (kernel) {
        case B200FP8_KERNEL_CTA1_N256:
            return depth == 2 ? B200FP8_LAUNCH5(256, 2, 1, 1, 2) : B200FP8_LAUNCH5(256, 4, 1, 1, 1);
        case B200FP8_KERNEL_CTA1_N128:
            return depth == 2 ? B200FP8_LAUNCH5(128, 2, 1, 1, 3) : depth == 4 ? B200FP8_LAUNCH5(128, 4, 1, 1, 1) : B200FP8_LAUNCH5(128, 6, 1, 1, 1);
        case B200FP8_KERNEL_PAIR_N256:
            return depth == 2 ? B200FP8_LAUNCH5(256, 2, 2, 1, 3) : depth == 4 ? B200FP8_LAUNCH5(256, 4, 2, 1, 1) : B200FP8_LAUNCH5(256, 6, 2, 1, 1);
        case B200FP8_KERNEL_CTA1_N64:
            // at most 64 rows and no sparse A: the short A box (16 / 32 / 64 rows), 18 / 16 / 12 k-blocks of B in flight
            if (depth == 0 && !ell && m <= 16) return B200FP8_LAUNCH6(64, 9, 1, 1, 2, 16);
            if (depth == 0 && !ell && m <= 32) return B200FP8_LAUNCH6(64, 8, 1, 1, 2, 32);
            if (depth == 0 && !ell && m <= 64) return B200FP8_LAUNCH6(64, 6, 1, 1, 2, 64);
            return depth == 2 ? B200FP8_LAUNCH5(64, 2, 1, 1, 4) : depth == 4 ? B200FP8_LAUNCH5(64, 4, 1, 1, 2) : B200FP8_LAUNCH5(64, 8, 1, 1, 1);
        case B200FP8_KERNEL_PAIR_N128:
            return depth == 2 ? B200FP8_LAUNCH5(128, 2, 2, 1, 4) : depth == 4 ? B200FP8_LAUNCH5(128, 4, 2, 1, 2) : B200FP8_LAUNCH5(128, 8, 2, 1, 1);
        case B200FP8_KERNEL_PAIR_N512:
            return depth == 2 ? B200FP8_LAUNCH5(256, 2, 2, 2, 2) : B200FP8_LAUNCH5(256, 4, 2, 2, 1);
        case B200FP8_KERNEL_SKINNY: {
            if (split_k > kSkinnyMaxSplits) return cudaErrorInvalidValue;
            long long* trace = nullptr;
#ifdef B200FP8_DIAGNOSTICS
            if ((tune().debug & 1024) && static_cast<long long>((n + kSkinnyTileN - 1) / kSkinnyTileN) * 8 * 8 <= kTraceWords)
                trace = trace_buffer();                          // eight time stamps per CTA
#endif
            e = launch_skinny(ctx->sm_count, ctx->status, g_encode, m, k, n, a, lda, b, ldb, c, ldc, a_dtype, b_dtype,
                              depth, split_k, epi, stream, nullptr, 0, trace, tune().pdl);
            if (e == cudaSuccess) ++t_launches;
            return e;
        }
        case B200FP8_KERNEL_SKINNY_STREAMK: {
            float4* scratch = nullptr;
            unsigned int* flags = nullptr;
            if ((e = streamk_slot(*ctx, &scratch, &flags)) != cudaSuccess) return e;
            long long* trace = nullptr;
#ifdef B200FP8_DIAGNOSTICS
            if ((tune().debug & 1024) && ctx->sm_count * 8 <= kTraceWords) trace = trace_buffer();
#endif
            e = launch_skinny_streamk(ctx->sm_count, ctx->status, scratch, flags, g_encode, m, k, n, a, lda, b, ldb, c, ldc,
                                      a_dtype, b_dtype, depth, split_k, epi, stream, nullptr, 0, trace, tune().pdl);
            if (e == cudaSuccess) ++t_launches;
            return e;
        }
        default:
            return cudaErrorInvalidValue;
    }
#undef B200FP8_LAUNCH5
#undef B200FP8_LAUNCH6
}

cudaError_t ensure(void** p, size_t* have, size_t want) {
    if (*have >= want) return cudaSuccess;
    if (*p) { cudaFree(*p); *p = nullptr; *have = 0; }
    cudaError_t e = cudaMalloc(p, want);
    if (e == cudaSuccess) *have = want;
    return e;
}

}  // namespace
}  // namespace b200fp8

using namespace b200fp8;

extern "C" {

int b200fp8_gemm_rowcol_f32(int m, int k, int n, const void* a, int a_dtype, const void* b, int b_dtype, float* c,
                            int depth, void* stream) {
    b200fp8_options opt{};
    opt.struct_bytes = sizeof(opt);
    opt.depth = depth;
    return gemm_dispatch(m, k, n, a, a_dtype, k, b, b_dtype, k, c, n, &opt, static_cast<cudaStream_t>(stream));
}

int b200fp8_gemm_rowcol_f32_ex(int m, int k, int n, const void* a, int a_dtype, long long lda, const void* b,
                               int b_dtype, long long ldb, float* c, long long ldc, const b200fp8_options* options,
                               void* stream) {
    if (options && options->struct_bytes != static_cast<int>(sizeof(b200fp8_options))) return cudaErrorInvalidValue;
    return gemm_dispatch(m, k, n, a, a_dtype, lda, b, b_dtype, ldb, c, ldc, options, static_cast<cudaStream_t>(stream));
}

int b200fp8_gemm_rowcol_scaled(int m, int k, int n, const void* a, int a_dtype, long long lda, const void* b, int b_dtype,
                               long long ldb, void* d, int d_dtype, long long ldd, float alpha, float beta,
                               const float* a_scale, const float* b_scale, const b200fp8_options* options, void* stream) {
    if (options && options->struct_bytes != static_cast<int>(sizeof(b200fp8_options))) return cudaErrorInvalidValue;
    if (d_dtype < B200FP8_OUT_F32 || d_dtype > B200FP8_OUT_F16) return cudaErrorInvalidValue;
    Epilogue epi{};
    epi.active = 1;
    epi.out_dtype = d_dtype;
    epi.alpha = alpha;
    epi.beta = beta;
    epi.a_scale = a_scale;
    epi.b_scale = b_scale;
    return gemm_dispatch(m, k, n, a, a_dtype, lda, b, b_dtype, ldb, static_cast<float*>(d), ldd, options,
                         static_cast<cudaStream_t>(stream), nullptr, &epi);
}

int b200fp8_gemm_rowcol_epilogue(int m, int k, int n, const void* a, int a_dtype, long long lda, const void* b,
                                 int b_dtype, long long ldb, void* d, int d_dtype, long long ldd,
                                 const b200fp8_epilogue* ep, const b200fp8_options* options, void* stream) {
    if (options && options->struct_bytes != static_cast<int>(sizeof(b200fp8_options))) return cudaErrorInvalidValue;
    if (!ep || (ep->struct_bytes != static_cast<int>(sizeof(b200fp8_epilogue)) && ep->struct_bytes != B200FP8_EPILOGUE_V1_BYTES))
        return cudaErrorInvalidValue;
    const bool extended = ep->struct_bytes == static_cast<int>(sizeof(b200fp8_epilogue));
    if (extended && (ep->activation < B200FP8_ACT_NONE || ep->activation > B200FP8_ACT_GELU_TANH)) return cudaErrorInvalidValue;
    if (d_dtype < B200FP8_OUT_F32 || d_dtype > B200FP8_OUT_E5M2) return cudaErrorInvalidValue;
    if (ep->bias && (ep->bias_dtype < B200FP8_OUT_F32 || ep->bias_dtype > B200FP8_OUT_F16)) return cudaErrorInvalidValue;
    if (ep->bias && (reinterpret_cast<uintptr_t>(ep->bias) % out_dtype_bytes(ep->bias_dtype))) return cudaErrorInvalidValue;
    if ((ep->amax_d && (reinterpret_cast<uintptr_t>(ep->amax_d) % 4)) || m < 0 || n < 0 || k <= 0) return cudaErrorInvalidValue;
    Epilogue epi{};
    epi.active = 1;
    epi.out_dtype = d_dtype;
    epi.alpha = ep->alpha;
    epi.beta = ep->beta;
    epi.a_scale = ep->a_scale;
    epi.b_scale = ep->b_scale;
    epi.d_scale = ep->d_scale;
    epi.amax = ep->amax_d;
    epi.bias = ep->bias;
    epi.bias_dtype = ep->bias_dtype;
    if (extended) {
        epi.activation = ep->activation;
        epi.a_row_scale = ep->a_row_scale;
        epi.b_row_scale = ep->b_row_scale;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (ep->amax_d) {                            // the kernel merges by atomic max: start from zero, stream-ordered
        cudaError_t e = cudaMemsetAsync(ep->amax_d, 0, sizeof(float), st);
        if (e != cudaSuccess) return e;
    }
    return gemm_dispatch(m, k, n, a, a_dtype, lda, b, b_dtype, ldb, static_cast<float*>(d), ldd, options, st, nullptr, &epi);
}

int b200fp8_gemv_f32(int n, int k, const void* b, int b_dtype, long long ldb, const void* x, int x_dtype, float* y,
                     void* stream) {
    // y[n] = sum_k B[n][k] x[k]: the operator with M = 1 (x is the single row of A), HBM-bound split-K kernel
    return gemm_dispatch(1, k, n, x, x_dtype, k, b, b_dtype, ldb, y, n, nullptr, static_cast<cudaStream_t>(stream));
}

int b200fp8_spmm_bell_rowcol_f32(int m, int k, int n, const void* ell_values, int a_dtype, long long lda,
                                 const int* ell_col_ind, int ell_blocks_per_row, const void* b, int b_dtype,
                                 long long ldb, float* c, long long ldc, const b200fp8_options* options, void* stream) {
    if (options && options->struct_bytes != static_cast<int>(sizeof(b200fp8_options))) return cudaErrorInvalidValue;
    if (k <= 0) return cudaErrorInvalidValue;
    EllSpec ell{ell_col_ind, ell_blocks_per_row};
    return gemm_dispatch(m, k, n, ell_values, a_dtype, lda, b, b_dtype, ldb, c, ldc, options,
                         static_cast<cudaStream_t>(stream), nullptr, nullptr, &ell);
}

int b200fp8_spmv_bell_f32(int m, int k, const void* ell_values, int a_dtype, long long lda, const int* ell_col_ind,
                          int ell_blocks_per_row, const void* x, int x_dtype, float* y, const b200fp8_options* options,
                          void* stream) {
    // y[m] = sum_k A[m][k] x[k] with A in blocked-ELL form: the split-K kernel with the roles swapped -- the sparse
    // matrix is the large, streamed operand (its block rows are the kernel's 128-row tiles), x the single small row
    if (options && options->struct_bytes != static_cast<int>(sizeof(b200fp8_options))) return cudaErrorInvalidValue;
    if (m < 0 || k <= 0 || ell_blocks_per_row < 0 || ell_blocks_per_row > (1 << 20) || !valid_dtype(a_dtype) ||
        !valid_dtype(x_dtype))
        return cudaErrorInvalidValue;
    if (m == 0) return cudaSuccess;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!y) return cudaErrorInvalidValue;
    if (ell_blocks_per_row == 0) return cudaMemsetAsync(y, 0, static_cast<size_t>(m) * sizeof(float), st);
    const long long width = static_cast<long long>(ell_blocks_per_row) * kBlockK;
    if (!ell_values || !ell_col_ind || !x || lda < width || (lda % 16) || (k % 16)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(ell_values) % 16) || (reinterpret_cast<uintptr_t>(x) % 16) ||
        (reinterpret_cast<uintptr_t>(y) % 4) || (reinterpret_cast<uintptr_t>(ell_col_ind) % 4))
        return cudaErrorInvalidValue;
    const int depth = options ? options->depth : 0;
    const int split_k = options ? options->split_k : 0;
    if ((depth != 0 && depth != 2 && depth != 4) || split_k < 0) return cudaErrorInvalidValue;
    DeviceCtx* ctx = nullptr;
    cudaError_t e = get_ctx(&ctx);
    if (e != cudaSuccess) return e;
    if (!(options && options->kernel == B200FP8_KERNEL_SKINNY_STREAMK)) {
        if (split_k > kSkinnyMaxSplits) return cudaErrorInvalidValue;
        e = launch_skinny(ctx->sm_count, ctx->status, g_encode, 1, static_cast<int>(width), m, x, k, ell_values, lda, y, m,
                          x_dtype, a_dtype, depth, split_k, nullptr, st, ell_col_ind, k, nullptr, tune().pdl);
    } else {
        if (split_k > 64) return cudaErrorInvalidValue;
        float4* scratch = nullptr;
        unsigned int* flags = nullptr;
        if ((e = streamk_slot(*ctx, &scratch, &flags)) != cudaSuccess) return e;
        e = launch_skinny_streamk(ctx->sm_count, ctx->status, scratch, flags, g_encode, 1, static_cast<int>(width), m, x, k,
                                  ell_values, lda, y, m, x_dtype, a_dtype, depth, split_k, nullptr, st, ell_col_ind, k,
                                  nullptr, tune().pdl);
    }
    if (e == cudaSuccess) ++t_launches;
    return e;
}

int b200fp8_gemm_rowcol_f32_allgather(int m, int k, int n_local, const void* a, int a_dtype, const void* b_shard,
                                      int b_dtype, float* const* c_all, float* c_multicast, int world, int rank,
                                      long long n_total, long long n_begin, const b200fp8_options* options,
                                      void* stream) {
    if (world < 1 || world > kMaxPeers + 1 || rank < 0 || rank >= world || !c_all) return cudaErrorInvalidValue;
    if (n_begin < 0 || n_local < 0 || n_begin + n_local > n_total || (n_begin % 4) || (n_total % 4)) return cudaErrorInvalidValue;
    if (options && options->struct_bytes != static_cast<int>(sizeof(b200fp8_options))) return cudaErrorInvalidValue;
    PeerSet peers;
    for (int r = 0; r < world; ++r)
        if (!c_all[r] || (reinterpret_cast<uintptr_t>(c_all[r]) % 16)) return cudaErrorInvalidValue;
    // every rank starts with its right-hand neighbour, so that at any moment the ranks store to different GPUs
    for (int i = 1; i < world; ++i) peers.c[peers.count++] = c_all[(rank + i) % world] + n_begin;
    if (c_multicast) {
        if (reinterpret_cast<uintptr_t>(c_multicast) % 16) return cudaErrorInvalidValue;
        peers.multicast = c_multicast + n_begin;
    }
    return gemm_dispatch(m, k, n_local, a, a_dtype, k, b_shard, b_dtype, k, c_all[rank] + n_begin, n_total, options,
                         static_cast<cudaStream_t>(stream), &peers);
}

int b200fp8_gemm_rowcol_f32_host(int m, int k, int n, const void* a_host, int a_dtype, const void* b_host, int b_dtype,
                                 float* c_host, int depth) {
    if (m < 0 || n < 0 || k < 0) return cudaErrorInvalidValue;
    if (m == 0 || n == 0) return cudaSuccess;
    if (!c_host || (k > 0 && (!a_host || !b_host))) return cudaErrorInvalidValue;
    DeviceCtx* ctx = nullptr;
    cudaError_t e = get_ctx(&ctx);
    if (e != cudaSuccess) return e;
    // one call at a time per device: the staging buffers and the three streams below belong to the call in progress
    std::lock_guard<std::mutex> host_lock(ctx->host_mutex);
    if (!ctx->compute) {
        if ((e = cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&ctx->compute, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking)) != cudaSuccess) return e;
    }
    const size_t a_bytes = static_cast<size_t>(m) * k, b_bytes = static_cast<size_t>(n) * k;
    const size_t c_bytes = static_cast<size_t>(m) * n * sizeof(float);
    if ((e = ensure(&ctx->host_a, &ctx->host_a_bytes, a_bytes ? a_bytes : 16)) != cudaSuccess) return e;
    if ((e = ensure(&ctx->host_b, &ctx->host_b_bytes, b_bytes ? b_bytes : 16)) != cudaSuccess) return e;
    if ((e = ensure(&ctx->host_c, &ctx->host_c_bytes, c_bytes)) != cudaSuccess) return e;
    float* dc = static_cast<float*>(ctx->host_c);
    const uint8_t* db = static_cast<const uint8_t*>(ctx->host_b);

    // Pipeline over a grid of C blocks so that uploads, the operator and the download of C overlap on three
    // streams.  C is the largest of the three matrices (4 bytes per element), so the call is bound by the
    // download of C and the goal is to start it as early as possible: operands go up in row blocks of A and
    // of B alternately (A0, B0, B1, A1, B2, A2, ...), and every C block is computed and sent down as soon as
    // its two operand blocks have arrived.  The first block needs 2 of the 2 x 8 uploads instead of a whole
    // operand, and the number of computable blocks grows quadratically while downloads drain them linearly.
    auto split = [](int extent, int want, int* step) {
        int blocks = want < 1 ? 1 : want;
        int st = ((extent + blocks - 1) / blocks + 255) / 256 * 256;
        if (st <= 0) st = extent;
        *step = st;
        return (extent + st - 1) / st;
    };
    constexpr int kMaxSide = 8;
    const bool big = static_cast<double>(m) * n * k > 1e11;
    int step_m = m, step_n = n;
    auto side = [&](int extent, int edge) { return extent < 2048 ? 1 : std::min(kMaxSide, (extent + edge - 1) / edge); };
    const int bm = big ? split(m, side(m, tune().host_block_m), &step_m) : 1;
    const int bn = big ? split(n, side(n, tune().host_block_n), &step_n) : 1;
    if (bm > kMaxSide || bn > kMaxSide) return cudaErrorInvalidValue;
    cudaEvent_t up_a[kMaxSide], up_b[kMaxSide], done[kMaxSide * kMaxSide];
    for (int i = 0; i < bm; ++i) cudaEventCreateWithFlags(&up_a[i], cudaEventDisableTiming);
    for (int j = 0; j < bn; ++j) cudaEventCreateWithFlags(&up_b[j], cudaEventDisableTiming);
    for (int t = 0; t < bm * bn; ++t) cudaEventCreateWithFlags(&done[t], cudaEventDisableTiming);
    b200fp8_options opt{};
    opt.struct_bytes = sizeof(opt);
    opt.depth = depth;
    cudaError_t first = cudaSuccess;
    auto keep = [&](cudaError_t x) { if (first == cudaSuccess && x != cudaSuccess) first = x; };
    uint8_t* da = static_cast<uint8_t*>(ctx->host_a);
    uint8_t* dbw = static_cast<uint8_t*>(ctx->host_b);
    const uint8_t* ha = static_cast<const uint8_t*>(a_host);
    const uint8_t* hb = static_cast<const uint8_t*>(b_host);
    auto rows_of = [](int idx, int step, int extent) { return extent - idx * step < step ? extent - idx * step : step; };
    auto upload = [&](bool is_a, int idx) {
        const int step = is_a ? step_m : step_n, rows = rows_of(idx, step, is_a ? m : n);
        const size_t off = static_cast<size_t>(idx) * step * k;
        if (k) keep(cudaMemcpyAsync((is_a ? da : dbw) + off, (is_a ? ha : hb) + off, static_cast<size_t>(rows) * k,
                                    cudaMemcpyHostToDevice, ctx->copy_in));
        keep(cudaEventRecord(is_a ? up_a[idx] : up_b[idx], ctx->copy_in));
    };
    auto block = [&](int i, int j, cudaEvent_t newest) {          // C block (i, j): operator, then its download
        const int mi = rows_of(i, step_m, m), nj = rows_of(j, step_n, n);
        const size_t c_off = static_cast<size_t>(i) * step_m * n + static_cast<size_t>(j) * step_n;
        keep(cudaStreamWaitEvent(ctx->compute, newest, 0));       // copy_in is ordered: the newest upload implies the older ones
        keep(gemm_dispatch(mi, k, nj, da + static_cast<size_t>(i) * step_m * k, a_dtype, k,
                           db + static_cast<size_t>(j) * step_n * k, b_dtype, k, dc + c_off, n, &opt, ctx->compute));
        cudaEvent_t d = done[i * bn + j];
        keep(cudaEventRecord(d, ctx->compute));
        keep(cudaStreamWaitEvent(ctx->copy_out, d, 0));
        keep(cudaMemcpy2DAsync(c_host + c_off, static_cast<size_t>(n) * 4, dc + c_off, static_cast<size_t>(n) * 4,
                               static_cast<size_t>(nj) * 4, mi, cudaMemcpyDeviceToHost, ctx->copy_out));
    };
    int na = 0, nb = 0;                                            // operand blocks uploaded so far
    upload(true, na++);
    upload(false, nb++);
    block(0, 0, up_b[0]);
    while ((na < bm || nb < bn) && first == cudaSuccess) {
        if (nb < bn && (nb <= na || na == bm)) {                   // next block of B: a new block column of C
            upload(false, nb);
            for (int i = 0; i < na; ++i) block(i, nb, up_b[nb]);
            ++nb;
        } else {                                                   // next block of A: a new block row of C
            upload(true, na);
            for (int j = 0; j < nb; ++j) block(na, j, up_a[na]);
            ++na;
        }
    }
    keep(cudaStreamSynchronize(ctx->copy_in));
    keep(cudaStreamSynchronize(ctx->compute));
    keep(cudaStreamSynchronize(ctx->copy_out));
    for (int i = 0; i < bm; ++i) cudaEventDestroy(up_a[i]);
    for (int j = 0; j < bn; ++j) cudaEventDestroy(up_b[j]);
    for (int t = 0; t < bm * bn; ++t) cudaEventDestroy(done[t]);
    return first;
}

int b200fp8_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                          void* stream) {
    if (rows == 0 || width_bytes == 0) return cudaSuccess;
    if (!dst || !src || dst_pitch < width_bytes || src_pitch < width_bytes) return cudaErrorInvalidValue;
    return cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault, static_cast<cudaStream_t>(stream));
}

int b200fp8_host_release(void) {
    DeviceCtx* ctx = nullptr;
    cudaError_t e = get_ctx(&ctx);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> host_lock(ctx->host_mutex);
    cudaError_t first = cudaSuccess;
    void** bufs[3] = {&ctx->host_a, &ctx->host_b, &ctx->host_c};
    size_t* sizes[3] = {&ctx->host_a_bytes, &ctx->host_b_bytes, &ctx->host_c_bytes};
    for (int i = 0; i < 3; ++i) {
        if (*bufs[i]) {
            e = cudaFree(*bufs[i]);
            if (first == cudaSuccess) first = e;
        }
        *bufs[i] = nullptr;
        *sizes[i] = 0;
    }
    return first;
}

// ---------------------------------------------------------------------------------------------
// b200fp8_gemm_rowcol_f32_noalloc: the pair kernels with their scratch memory in a static device
// array, for callers that must not allocate (see include/b200fp8.h).  Nothing on this path calls
// cudaMalloc / cudaFree or touches the library's per-device context, which owns allocated buffers.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace b200fp8 {
namespace {

constexpr int kNoAllocScratchWords = 64;                    // 256 bytes per GPU that loads the library
constexpr long long kNoAllocMaxTiles = 1LL << 24;           // tiles per call the pacing counter is specified for

// Word 0 is the tile-pacing counter of the pair kernels (must be zero when a launch starts).
// The remaining words are reserved.  Every call on a device shares this one array.
static __device__ __align__(256) unsigned int g_noalloc_scratch[kNoAllocScratchWords];

struct NoAllocDevice {
    bool ready = false;
    int sm_count = 0;
    unsigned int* scratch = nullptr;    // DEVICE address of g_noalloc_scratch on this device
};
NoAllocDevice g_noalloc[kMaxDevices];

template <int BN, int STAGES, int NACC>
cudaError_t noalloc_prepare_kernel() {
    return cudaFuncSetAttribute(gemm_fp8_rowcol_kernel<BN, STAGES, 2, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                GemmSmem<BN, STAGES, 2, NACC>::kDynamicBytes);
}

// One-time set-up per device, with that device current: resolves the device address of the static
// array (the array's name is only a host-side handle and must never be given to a kernel),
// raises the kernels' shared-memory limit and zeroes the array.
cudaError_t noalloc_device(NoAllocDevice** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    NoAllocDevice& d = g_noalloc[dev];
    if (!d.ready) {
        int major = 0;
        if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return e;
        if (major != 10) return cudaErrorNoKernelImageForDevice;
        if ((e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
        if ((e = load_encode()) != cudaSuccess) return e;
        void* ptr = nullptr;
        if ((e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch)) != cudaSuccess) return e;
        if ((e = noalloc_prepare_kernel<256, 6, 1>()) != cudaSuccess) return e;
        if ((e = noalloc_prepare_kernel<256, 4, 2>()) != cudaSuccess) return e;
        if ((e = cudaMemset(ptr, 0, sizeof(unsigned int) * kNoAllocScratchWords)) != cudaSuccess) return e;
        d.scratch = static_cast<unsigned int*>(ptr);
        d.ready = true;
    }
    *out = &d;
    return cudaSuccess;
}

template <int BN, int STAGES, int NACC>
cudaError_t noalloc_launch(const NoAllocDevice& d, int m, int k, int n, const void* a, const void* b, float* c,
                           int a_dtype, int b_dtype, int* status_word, cudaStream_t stream) {
    using L = GemmSmem<BN, STAGES, 2, NACC>;
    GemmArgs args{};
    args.M = m; args.N = n; args.K = k;
    args.num_k_blocks = (k + kBlockK - 1) / kBlockK;
    args.m_tiles = (m + 2 * kTileM - 1) / (2 * kTileM);
    args.n_tiles = (n + L::kTileN - 1) / L::kTileN;
    args.group_m = 16;
    args.idesc = make_idesc_f8(a_dtype, b_dtype, 2 * kTileM, BN);
    args.tma_store = ((n % 4) == 0 && (reinterpret_cast<uintptr_t>(c) % 16) == 0) ? 1 : 0;
    args.C = c; args.ldc = n; args.status = status_word;
    const long long tiles = static_cast<long long>(args.m_tiles) * args.n_tiles;
    if (tiles > kNoAllocMaxTiles) {
        fprintf(stderr, "b200fp8_gemm_rowcol_f32_noalloc: %lld output tiles exceed the maximum of %lld this entry point supports\n",
                tiles, kNoAllocMaxTiles);
        return cudaErrorInvalidValue;
    }
    CUtensorMap ta, tb, tc;
    cudaError_t e;
    if ((e = encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, k, m, k, kBlockK, kTileM)) != cudaSuccess) return e;
    if ((e = encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, k, n, k, kBlockK, L::kBRows)) != cudaSuccess) return e;
    if (args.tma_store) {
        if ((e = encode_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, c, n, m, n, 32, 32)) != cudaSuccess) return e;
    } else {
        tc = ta;
    }
    int units = d.sm_count / 2;
    if (tiles < units) units = static_cast<int>(tiles);
    args.full_items = static_cast<int>(tiles);
    args.split_tiles = 0;
    if (tiles >= 8LL * units) {
        // the counter keeps whatever the previous call left: it has to start from zero
        if ((e = cudaMemsetAsync(d.scratch, 0, sizeof(unsigned int), stream)) != cudaSuccess) return e;
        args.pace = d.scratch;
        args.pace_limit_ns = 30000;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(units * 2), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynamicBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, gemm_fp8_rowcol_kernel<BN, STAGES, 2, NACC>, ta, tb, tc, tb, args);
    if (e == cudaSuccess) ++t_launches;
    return e;
}

}  // namespace
}  // namespace b200fp8

extern "C" {

int b200fp8_gemm_rowcol_f32_noalloc(int m, int k, int n, const void* a, int a_dtype, const void* b, int b_dtype,
                                    float* c, int* status_word, void* stream) {
    if (m < 0 || n < 0 || k < 0 || !valid_dtype(a_dtype) || !valid_dtype(b_dtype)) return cudaErrorInvalidValue;
    if (m == 0 || n == 0) return cudaSuccess;
    if (!c || !a || !b || k == 0 || (k % 16)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(a) % 16) || (reinterpret_cast<uintptr_t>(b) % 16) ||
        (reinterpret_cast<uintptr_t>(c) % 4) || (reinterpret_cast<uintptr_t>(status_word) % 4))
        return cudaErrorInvalidValue;
    NoAllocDevice* d = nullptr;
    cudaError_t e = noalloc_device(&d);
    if (e != cudaSuccess) return e;
    const long long wide_tiles = static_cast<long long>((m + 255) / 256) * ((n + 511) / 512);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (wide_tiles >= 16LL * (d->sm_count / 2) && k >= 8192)
        return noalloc_launch<256, 4, 2>(*d, m, k, n, a, b, c, a_dtype, b_dtype, status_word, s);
    return noalloc_launch<256, 6, 1>(*d, m, k, n, a, b, c, a_dtype, b_dtype, status_word, s);
}

int b200fp8_fill_normal(void* dst, long long count, int dtype, float sigma, unsigned long long seed,
                        unsigned long long index_offset, void* stream) {
    if (count < 0 || !valid_dtype(dtype) || (count > 0 && !dst)) return cudaErrorInvalidValue;
    if (count == 0) return cudaSuccess;
    DeviceCtx* ctx = nullptr;
    cudaError_t e = get_ctx(&ctx);
    if (e != cudaSuccess) return e;
    e = launch_fill_normal(static_cast<uint8_t*>(dst), count, dtype, sigma, seed, index_offset, ctx->sm_count,
                           static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) ++t_launches;
    return e;
}

int b200fp8_device_status(int* status, int reset) {
    if (!status) return cudaErrorInvalidValue;
    DeviceCtx* ctx = nullptr;
    cudaError_t e = get_ctx(&ctx);
    if (e != cudaSuccess) return e;
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e;
    if ((e = cudaMemcpy(status, ctx->status, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess) return e;
    if (reset) e = cudaMemset(ctx->status, 0, sizeof(int));
    if (reset && *status != 0) {
        // a kernel that gave up may have left stream-K flags raised: the next launch must find them zero
        std::lock_guard<std::mutex> lock(g_mutex);
        for (int i = 0; i < StreamKWorkspace::kSlots && ctx->streamk.max_ctas > 0; ++i)
            cudaMemset(ctx->streamk.flags[i], 0, ctx->streamk.max_ctas * sizeof(unsigned int));
    }
    return e;
}

int b200fp8_enable_peer_access(int peer_device) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (peer_device == dev) return cudaSuccess;
    int can = 0;
    if ((e = cudaDeviceCanAccessPeer(&can, dev, peer_device)) != cudaSuccess) return e;
    if (!can) return cudaErrorPeerAccessUnsupported;
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
    return e;
}

int b200fp8_ipc_alloc(size_t bytes, void** device_ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!device_ptr || !handle || bytes == 0) return cudaErrorInvalidValue;
    cudaError_t e = cudaMalloc(device_ptr, bytes);
    if (e != cudaSuccess) return e;
    cudaIpcMemHandle_t h;
    if ((e = cudaIpcGetMemHandle(&h, *device_ptr)) != cudaSuccess) { cudaFree(*device_ptr); *device_ptr = nullptr; return e; }
    memcpy(handle, &h, sizeof(h));
    return cudaSuccess;
}

int b200fp8_ipc_open(const unsigned char handle[64], void** device_ptr) {
    if (!device_ptr || !handle) return cudaErrorInvalidValue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    // opened with the IMPORTING device current: the mapping is made for this device, peer access enabled lazily
    return cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

int b200fp8_ipc_close(void* device_ptr) { return device_ptr ? cudaIpcCloseMemHandle(device_ptr) : cudaSuccess; }

int b200fp8_ipc_free(void* device_ptr) { return device_ptr ? cudaFree(device_ptr) : cudaSuccess; }

long long b200fp8_launch_count(void) { return t_launches; }

int b200fp8_choose_kernel(int m, int k, int n) {
    DeviceCtx* ctx = nullptr;
    if (m <= 0 || n <= 0 || k < 0 || get_ctx(&ctx) != cudaSuccess) return -1;
    return choose_kernel(ctx->sm_count, m, k, n, false);
}

int b200fp8_l2_sides(unsigned long long mask[3]) {
    DeviceCtx* ctx = nullptr;
    if (mask) mask[0] = mask[1] = mask[2] = 0;
    if (get_ctx(&ctx) != cudaSuccess || !ctx->sides_known) return 0;
    int count = 0;
    for (int i = 0; i < 3; ++i) {
        if (mask) mask[i] = ctx->side_mask[i];
        count += __builtin_popcountll(ctx->side_mask[i]);
    }
    return count;
}

#ifdef B200FP8_DIAGNOSTICS
// diagnostics build only (declared in include/b200fp8.h under the same macro)
void* b200fp8_debug_trace(void) { return g_trace; }

// copies the first `count` trace words to the host (after a device synchronise) and, with
// `clear`, zeroes the device buffer for the next launch.  Returns the number of words copied (0: no trace).
int b200fp8_debug_trace_copy(long long* dst, int count, int clear) {
    if (!g_trace || !dst || count <= 0) return 0;
    if (count > kTraceWords) count = kTraceWords;
    if (cudaDeviceSynchronize() != cudaSuccess) return 0;
    if (cudaMemcpy(dst, g_trace, static_cast<size_t>(count) * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
    if (clear) cudaMemset(g_trace, 0, kTraceWords * sizeof(long long));
    return count;
}
#endif

const char* b200fp8_version(void) { return "b200fp8 0.1 sm_100a"; }

}  // extern "C"
