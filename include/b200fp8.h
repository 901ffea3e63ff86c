/*
 * b200fp8 -- C ABI of the B200 (sm_100a) FP8 GEMM library.
 *
 * The operation is the one behind the reference project's operator API
 * (xuezy-mmi/Tensor-Core-FP8, GEMM/include/gemm.cuh:12-55):
 *
 *     C[m][n] = sum_k A[m][k] * B[n][k]          "row-col" layout
 *
 * A is row-major M x K, B is "column-major K x N", i.e. stored as N rows of K
 * contiguous elements, both 8-bit floats (e4m3 or e5m2, any of the four
 * combinations); C is row-major M x N FP32, fully overwritten.  No alpha/beta,
 * no scaling.  All matrix pointers are DEVICE pointers owned by the caller
 * unless an entry point says otherwise; calls are asynchronous with respect to
 * the host and ordered on the given stream, like the reference's launchers
 * (GEMM/src/gemm.cu:263-277).
 *
 * Every function returns a cudaError_t value as int: 0 (cudaSuccess),
 * 1 (cudaErrorInvalidValue) for bad arguments -- nothing is launched in that
 * case -- or the CUDA error of the failing runtime call.  Nothing here aborts,
 * throws or exits.
 *
 * Requirements of the tensor-core path: A, B 16-byte aligned, K (and lda, ldb)
 * multiples of 16.  M and N are arbitrary (ragged edges are clipped in
 * hardware).  The reference itself needs M, N multiples of 128 and K a
 * multiple of 64 (GEMM/src/gemm.cu:45-47, :117).
 */
#ifndef B200FP8_H
#define B200FP8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 8-bit float formats (cuda_fp8.h: __nv_fp8_e4m3 / __nv_fp8_e5m2, typedef'd
 * e4m3 / e5m2 in GEMM/include/gemm.cuh:6-7). */
enum { B200FP8_E4M3 = 0, B200FP8_E5M2 = 1 };

/* Kernel selection for b200fp8_options.kernel */
enum {
    B200FP8_KERNEL_AUTO = 0,
    B200FP8_KERNEL_CTA1_N256 = 1, /* one CTA per 128x256 tile                       */
    B200FP8_KERNEL_CTA1_N128 = 2, /* one CTA per 128x128 tile                       */
    B200FP8_KERNEL_PAIR_N256 = 3, /* CTA pair (cta_group::2) per 256x256 tile       */
    B200FP8_KERNEL_SKINNY = 4,    /* swap-AB split-K kernel for M <= 128, K splits of a tile in one cluster */
    B200FP8_KERNEL_PAIR_N512 = 5, /* CTA pair per 256x512 tile: least traffic per flop */
    B200FP8_KERNEL_PAIR_N128 = 6, /* CTA pair per 256x128 tile: 128 < M <= 256 with a large N */
    B200FP8_KERNEL_CTA1_N64 = 7,  /* one CTA per 128x64 tile: twice the CTAs for problems of a few tiles */
    B200FP8_KERNEL_SKINNY_STREAMK = 8 /* swap-AB stream-K kernel for M <= 128: every SM streams the same share of B,
                                         partial tiles meet in L2; never chosen automatically (measured slower
                                         than kernel 4 on B200), kept selectable */
};

typedef struct b200fp8_options {
    int struct_bytes; /* sizeof(b200fp8_options), for forward compatibility          */
    int depth;        /* shared-memory ring depth: 2, 4, or 0 = as deep as fits      */
    int kernel;       /* B200FP8_KERNEL_*                                            */
    int split_k;      /* skinny kernels: number of K splits (kernel 4, <= 8) / most pieces
                         a tile's K range is cut into (kernel 8, <= 64); 0 = automatic */
    int max_ctas;     /* cap on the persistent grid (0 = one CTA per SM); testing    */
} b200fp8_options;

/*
 * Replaces gemm::GEMM (depth = 2) and gemm::GEMM4 (depth = 4), all four dtype
 * overloads: decl GEMM/include/gemm.cuh:12-55, def GEMM/src/gemm.cu:278-285,
 * :687-694, :937-944, :1192-1199, :1447-1454, :1479-1548.  Argument order
 * m, k, n as in the reference; lda = ldb = k, ldc = n.  `stream` is a
 * cudaStream_t (NULL = the legacy default stream the reference launches on).
 */
int b200fp8_gemm_rowcol_f32(int m, int k, int n, const void* a, int a_dtype, const void* b, int b_dtype,
                            float* c, int depth, void* stream);

/*
 * Same operation with explicit leading dimensions (in elements) and options.
 * ldc lets a rank of an N-sharded run write its column block in place inside a
 * full M x N matrix.  Extends the launchers GEMMex / GEMMex4
 * (GEMM/src/gemm.cu:263-277, :670-686), which take no options.
 */
int b200fp8_gemm_rowcol_f32_ex(int m, int k, int n, const void* a, int a_dtype, long long lda, const void* b,
                               int b_dtype, long long ldb, float* c, long long ldc, const b200fp8_options* options,
                               void* stream);

/* Output types of b200fp8_gemm_rowcol_scaled (the first three) and b200fp8_gemm_rowcol_epilogue (all) */
enum { B200FP8_OUT_F32 = 0, B200FP8_OUT_BF16 = 1, B200FP8_OUT_F16 = 2, B200FP8_OUT_E4M3 = 3, B200FP8_OUT_E5M2 = 4 };

/*
 * The operator with the epilogue of the reference's cuBLASLt comparator
 * (GEMM/src/cublas.cu:37-53, :79-88: alpha, beta, per-tensor scale pointers;
 * GEMM/src/matmul-fp8-v0.cu:109-111 writes FP16):
 *
 *     D = alpha * a_scale * b_scale * (A B^T) + beta * D
 *
 * D is M x N with row pitch ldd, FP32, BF16 or FP16 (`d_dtype`), read only when
 * beta != 0 and updated in place.  `a_scale` / `b_scale` are optional DEVICE
 * scalars (NULL = 1), read by the kernel, so a producer on the same stream may
 * still be computing them when this call is enqueued.  Layouts, dtypes and
 * requirements of A and B as for the plain operator; D must be aligned to its
 * element size (16 bytes and ldd * element size a multiple of 16 for the fast
 * store path).  K must be positive.
 */
int b200fp8_gemm_rowcol_scaled(int m, int k, int n, const void* a, int a_dtype, long long lda, const void* b, int b_dtype,
                               long long ldb, void* d, int d_dtype, long long ldd, float alpha, float beta,
                               const float* a_scale, const float* b_scale, const b200fp8_options* options, void* stream);

/*
 * Full epilogue of the reference's cuBLASLt comparator: what the call above does,
 * plus the output scale, the absolute maximum and a bias vector, and 8-bit output
 * (GEMM/src/cublas.cu:37-53 sets A/B/D scale pointers on the matmul descriptor;
 * GEMM/include/helper.h:59-66 carries the amax and scale slots):
 *
 *     t      = act(alpha * a_scale * b_scale * a_row_scale[m] * b_row_scale[n] * (A B^T) + beta * D + bias[n])
 *     amax_d = max over the M x N result of |t|          (NaNs are ignored)
 *     D      = convert(d_scale * t)
 *
 * a_row_scale (M floats, one per row of A) and b_row_scale (N floats, one per row of
 * B) are the per-row scales of row-wise quantised operands (cuBLASLt's outer-vector
 * scaling mode); they multiply the per-tensor scalars.  act is one of
 * B200FP8_ACT_* and follows the bias, like cuBLASLt's RELU_BIAS / GELU_BIAS
 * epilogues; amax_d sees the activated value.  Scales that vary along K (blocks of 32
 * or 128 elements of K) are not offered: they cannot be applied after the sum.
 *
 * d_dtype: any B200FP8_OUT_*.  8-bit outputs round to nearest even and saturate to
 * the largest finite value (448 for E4M3, 57344 for E5M2), as the toolkit's host
 * conversions do.  With beta != 0 the old D is read in d_dtype.  All pointers in
 * the struct are DEVICE pointers and optional (NULL = scale 1 / no amax / no bias).
 * amax_d is zeroed on `stream` before the kernel and written by atomic max, so it
 * is complete when the kernel has finished.  bias holds N values of bias_dtype
 * (B200FP8_OUT_F32, _BF16 or _F16).  K must be positive.
 */
typedef struct b200fp8_epilogue {
    int struct_bytes;      /* sizeof(b200fp8_epilogue) */
    float alpha, beta;
    const float* a_scale;
    const float* b_scale;
    const float* d_scale;
    float* amax_d;
    const void* bias;
    int bias_dtype;
    /* fields below: present when struct_bytes == sizeof(b200fp8_epilogue); a caller compiled against the shorter
       struct (struct_bytes == B200FP8_EPILOGUE_V1_BYTES) gets no row scales and no activation */
    int activation;            /* B200FP8_ACT_* */
    const float* a_row_scale;  /* M values or NULL */
    const float* b_row_scale;  /* N values or NULL */
} b200fp8_epilogue;

/* RELU keeps NaNs.  GELU_ERF = 0.5 t (1 + erf(t / sqrt 2)), GELU_TANH = 0.5 t (1 + tanh(sqrt(2/pi) (t + 0.044715 t^3))),
   both by short branch-free FP32 formulas: within 2e-6 relative of the exact function for t >= 0 and within
   1e-6 |t| absolute for t < 0 (where the exact value itself falls below that). */
enum { B200FP8_ACT_NONE = 0, B200FP8_ACT_RELU = 1, B200FP8_ACT_GELU_ERF = 2, B200FP8_ACT_GELU_TANH = 3 };
/* sizeof(b200fp8_epilogue) before `activation` was added: the struct then ended with bias_dtype and its tail padding,
   where `activation` now sits */
#define B200FP8_EPILOGUE_V1_BYTES \
    ((int)((offsetof(b200fp8_epilogue, activation) + sizeof(void*) - 1) / sizeof(void*) * sizeof(void*)))

int b200fp8_gemm_rowcol_epilogue(int m, int k, int n, const void* a, int a_dtype, long long lda, const void* b,
                                 int b_dtype, long long ldb, void* d, int d_dtype, long long ldd,
                                 const b200fp8_epilogue* epilogue, const b200fp8_options* options, void* stream);

/*
 * GEMV, SpMM and SpMV: the next kernels on the reference's roadmap (README.md:7, "GEMM,
 * GEMV, SpMM, SpMV"); the reference ships only their input generators
 * (GEMM/include/bm_test_utils.h:48-70 blocked-ELL column indices, :73-130 CSR) and no
 * kernels, so these entry points have no counterpart to replace.
 *
 * b200fp8_gemv_f32:  y[n] = sum_k B[n][k] * x[k]  -- the operator with M = 1.
 *
 * Blocked-ELL sparse A, the format of GenerateUniformBlockedELLIndex
 * (bm_test_utils.h:48-70) with 128 x 128 blocks: every block row (128 rows of A) stores
 * `ell_blocks_per_row` blocks; `ell_values` is the compact row-major matrix
 * [M][ell_blocks_per_row * 128] (pitch lda, 8-bit floats) and
 * `ell_col_ind[ceil(M/128)][ell_blocks_per_row]` (DEVICE, int32) gives for each block the
 * block column of A it occupies, i.e. columns [128*c, 128*c + 128) of K.  An index < 0 or
 * beyond K marks a padding block that contributes nothing, whatever its values.  Blocks
 * are accumulated in stored order.
 *
 * b200fp8_spmm_bell_rowcol_f32:  C[M][N] = A_sparse[M][K] * B[N][K]^T   (B, C as in the dense operator;
 *                                options->kernel: AUTO, CTA1_N256 or CTA1_N128)
 * b200fp8_spmv_bell_f32:         y[M]    = A_sparse[M][K] * x[K]          (options->kernel: AUTO, SKINNY or SKINNY_STREAMK)
 */
int b200fp8_gemv_f32(int n, int k, const void* b, int b_dtype, long long ldb, const void* x, int x_dtype, float* y,
                     void* stream);
int b200fp8_spmm_bell_rowcol_f32(int m, int k, int n, const void* ell_values, int a_dtype, long long lda,
                                 const int* ell_col_ind, int ell_blocks_per_row, const void* b, int b_dtype,
                                 long long ldb, float* c, long long ldc, const b200fp8_options* options, void* stream);
int b200fp8_spmv_bell_f32(int m, int k, const void* ell_values, int a_dtype, long long lda, const int* ell_col_ind,
                          int ell_blocks_per_row, const void* x, int x_dtype, float* y, const b200fp8_options* options,
                          void* stream);

/*
 * N-sharded multi-GPU GEMM with the all-gather of C fused into the kernel's
 * epilogue (no counterpart in the reference, which is single-GPU; it follows
 * the operator above).  Rank `rank` of `world` (<= 8, one process per GPU)
 * owns rows [n_begin, n_begin + n_local) of B -- `b_shard` points at them --
 * and computes the matching column block of C.  `c_all` is a HOST array of
 * `world` DEVICE pointers: the full M x n_total matrix C of every rank, own
 * included; the other ranks' matrices must be mapped into this process (CUDA
 * IPC, peer access enabled).  Every finished 32x32 box of the block is stored
 * to the own matrix and, with plain 16-byte stores over NVLink, to the same
 * position of every peer's matrix, so that after all ranks' kernels have
 * finished each rank holds the complete row-major C: no separate collective
 * and no re-layout pass.  Requirements on top of the operator's: n_total and
 * n_begin multiples of 4, every C base 16-byte aligned.  The caller
 * synchronises the ranks (stream sync + barrier) before reading C.
 * `c_multicast`, when not NULL, is an NVSwitch multicast address bound to the same matrices (all ranks'
 * C at the same offsets): the epilogue then issues ONE multimem store per 16 bytes, which the switch
 * delivers to every rank's matrix including the own, instead of one store per peer.
 */
int b200fp8_gemm_rowcol_f32_allgather(int m, int k, int n_local, const void* a, int a_dtype, const void* b_shard,
                                      int b_dtype, float* const* c_all, float* c_multicast, int world, int rank,
                                      long long n_total, long long n_begin, const b200fp8_options* options,
                                      void* stream);

/*
 * The N-sharded GEMM over the GPUs of one box from ONE process: a plan object for C and C++
 * callers (the reference's caller is a C++ program, GEMM/gemm_main.cpp:28-194; the reference
 * itself is single-GPU, so these entry points have no counterpart to replace -- each shard
 * runs the operator of GEMM/include/gemm.cuh:12-55 on its slab).
 *
 * Shard i of `num_shards` (<= 8) runs on CUDA device devices[i] and owns an even share of B's
 * rows in units of 256 (rows [n_begin_i, n_end_i) of B = the same columns of C); A is
 * replicated.  The compute step exchanges nothing.  Inside b200fp8_multi_run one host thread
 * per shard enqueues `steps` operator calls on the shard's own stream, the threads start
 * together, and *max_ms_per_step is the MAXIMUM over the shards of the device time per step.
 * With `gather` != 0 every shard's C is the full M x N matrix and the kernels' epilogues
 * store every finished box into all of them (b200fp8_gemm_rowcol_f32_allgather; peer access
 * between the devices is enabled by b200fp8_multi_create; N must be a multiple of 4), so after
 * the call every device holds the complete row-major C.  A device may appear more than once
 * in `devices` (several shards on one GPU).
 *
 * b200fp8_multi_upload:      A (M x K) to every shard and B's slabs from HOST matrices (B is N x K).
 * b200fp8_multi_fill_normal: the same operands generated on the devices (b200fp8_fill_normal;
 *                            shard i generates exactly its slab of the full B).
 * b200fp8_multi_download:    the row-major M x N result into c_host -- the column blocks of all
 *                            shards, or with gather the full matrix of shard `from_shard`.
 * b200fp8_multi_shard:       a shard's device, column range and DEVICE pointers (any out-pointer
 *                            may be NULL); *ldc is C's row pitch in elements.
 * b200fp8_multi_destroy:     waits for the shards' streams, then frees everything.
 */
typedef struct b200fp8_multi b200fp8_multi;
int b200fp8_multi_create(int num_shards, const int* devices, int m, int k, int n, int a_dtype, int b_dtype, int gather,
                         b200fp8_multi** plan);
int b200fp8_multi_destroy(b200fp8_multi* plan);
int b200fp8_multi_shard(const b200fp8_multi* plan, int shard, int* device, long long* n_begin, long long* n_end, void** a,
                        void** b, float** c, long long* ldc);
int b200fp8_multi_upload(b200fp8_multi* plan, const void* a_host, const void* b_host);
int b200fp8_multi_fill_normal(b200fp8_multi* plan, float sigma_a, unsigned long long seed_a, float sigma_b,
                              unsigned long long seed_b);
int b200fp8_multi_run(b200fp8_multi* plan, int steps, const b200fp8_options* options, float* max_ms_per_step);
int b200fp8_multi_download(b200fp8_multi* plan, float* c_host, int from_shard);

/*
 * The whole call sequence of the reference's benchmark driver for one GEMM
 * (BmFN, GEMM/gemm_main.cpp:56-64 upload, :77 / :123 operator call, :161
 * download) with HOST pointers: uploads A and B, runs the operator, downloads
 * C, and returns when C is complete in host memory.  Device buffers are owned
 * by the library and reused between calls.  Copies overlap the computation in
 * column blocks of B / C.  Pinned host memory makes the copies asynchronous.
 */
int b200fp8_gemm_rowcol_f32_host(int m, int k, int n, const void* a_host, int a_dtype, const void* b_host,
                                 int b_dtype, float* c_host, int depth);

/*
 * Frees the device staging buffers b200fp8_gemm_rowcol_f32_host keeps on the current
 * device between calls (they grow to the largest problem seen: A, B and C of it).  The
 * next call allocates again.  Waits for a call in progress on this device.
 */
int b200fp8_host_release(void);

/*
 * A pitched copy, enqueued on `stream`: `rows` rows of `width_bytes` bytes from `src` (row pitch `src_pitch` bytes) to
 * `dst` (row pitch `dst_pitch`), between device memory and pinned host memory in either direction (cudaMemcpy2DAsync
 * with the direction taken from the pointers).  What the host-pointer entry above uses for its blocks of C; exported
 * for callers that pipeline column blocks of a row-major matrix themselves (the multi-GPU host driver does).
 * No counterpart in the reference.
 */
int b200fp8_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                          void* stream);

/*
 * Thread safety.  Every entry point may be called from several host threads at once, on the
 * same or on different devices.  Calls of b200fp8_gemm_rowcol_f32_host on ONE device are
 * serialised inside the library (they share that device's staging buffers and copy streams);
 * the device-pointer entry points only enqueue work and share nothing but the small scratch
 * rings described in INTEGRATION.md.
 */

/*
 * Seeded synthetic operands: element i (i counted from index_offset) becomes
 * fp8(sigma * z_i), z_i ~ N(0,1) from a counter-based generator keyed by
 * (seed, index), cast with round-to-nearest-even and saturate-to-finite -- the
 * conversion of the FP8 constructors the reference's MakeDenseMatrix uses
 * (GEMM/include/bm_test_utils.h:131-143); the distribution replaces its
 * uniform(-1,1).  A shard regenerates its slice from index_offset alone.
 */
int b200fp8_fill_normal(void* dst, long long count, int dtype, float sigma, unsigned long long seed,
                        unsigned long long index_offset, void* stream);

/*
 * Device status word of the current device: 0 when every kernel of this
 * library ran its pipeline to completion, otherwise the first recorded code
 * (a bounded wait inside a kernel ran out).  Synchronises the device.  `reset`
 * non-zero clears the word after reading.  The reference has no counterpart:
 * its kernels cannot report anything (GEMM/src/gemm.cu:276 returns only the
 * launch status).
 */
int b200fp8_device_status(int* status, int reset);

/*
 * The same GEMM (lda = ldb = k, ldc = n) for callers that are not allowed to
 * allocate device memory.  This entry point has no counterpart in the
 * reference.  Who needs it: a plugin loaded into a host program that reserved
 * the whole device for its own memory pool and forbids cudaMalloc behind its
 * back, a service with a hard per-process memory budget, or a latency-critical
 * loop that cannot take the device-wide synchronisation an allocation or a
 * free may imply.  The other entry points allocate a few small per-device
 * buffers on first use; this one calls no cudaMalloc, cudaFree or allocating
 * library routine, ever.
 *
 * Its scratch memory -- the counter the CTA-pair kernels use to keep their
 * tiles in step -- lives in a static 256-byte device array inside the
 * library (every GPU that loads the library holds those 256 bytes until the
 * process exits).  Consequences:
 *   - all calls on one device share that array: two calls whose kernels
 *     overlap on the GPU (different streams) race on it; issue them on one
 *     stream, or otherwise keep them from overlapping;
 *   - the first call on each device resolves the array's device address and
 *     prepares the kernels; make that first call outside any stream capture;
 *   - at most 2^24 output tiles per call (a tile is 256 x 256 elements, or
 *     256 x 512 for the large problems that take the wide-tile kernel); larger
 *     problems are rejected with cudaErrorInvalidValue and a message on stderr.
 * Always runs a CTA-pair kernel, whatever the shape.  `status_word` is an
 * optional DEVICE int the caller owns and has zeroed: a kernel whose bounded
 * wait runs out stores its code there (the role b200fp8_device_status plays
 * for the other entry points); pass NULL to do without.
 */
int b200fp8_gemm_rowcol_f32_noalloc(int m, int k, int n, const void* a, int a_dtype, const void* b, int b_dtype,
                                    float* c, int* status_word, void* stream);

/*
 * Lets kernels on the current device store into memory of `peer_device` (needed once per
 * peer before b200fp8_gemm_rowcol_f32_allgather; already-enabled counts as success).
 */
int b200fp8_enable_peer_access(int peer_device);

/*
 * Device memory that other processes on the same node can map (CUDA IPC), for the C matrices of
 * b200fp8_gemm_rowcol_f32_allgather.  The owner allocates and gets a 64-byte handle to hand to its
 * peers (any transport); a peer opens it WITH ITS OWN DEVICE CURRENT, which maps the memory for that
 * device and enables peer access as needed, and closes it before the owner frees.
 */
int b200fp8_ipc_alloc(size_t bytes, void** device_ptr, unsigned char handle[64]);
int b200fp8_ipc_open(const unsigned char handle[64], void** device_ptr);
int b200fp8_ipc_close(void* device_ptr);
int b200fp8_ipc_free(void* device_ptr);

/* Number of this library's kernels launched by the calling thread so far. */
long long b200fp8_launch_count(void);

/*
 * The kernel (a B200FP8_KERNEL_* id, never AUTO) that `kernel = AUTO` selects on the current device for a dense
 * M x K x N problem; -1 for an invalid shape or when the device cannot be used.  For tools that audit the rules
 * (time the selected kernel against the others) and for callers that want to log the choice.  No counterpart in the
 * reference, which has one kernel per operator.
 */
int b200fp8_choose_kernel(int m, int k, int n);

/*
 * How the current device's SMs divide over the two halves of its L2 (a B200 is two dies, each with half of the SMs
 * and half of the L2; which SM ids sit on which die differs between GPUs).  The library measures this once per device,
 * when the device is first used (two small kernels that time reads, a transient 16 MiB allocation), and gives the
 * CTA pairs of each die a contiguous run of tiles in long persistent runs, so that operand panels cross the
 * die-to-die link for one die instead of two.  B200FP8_DIE_AWARE=0 in the environment switches both off.
 * mask (three 64-bit words, optional): bit s is set when SM s sits on the second side, the first side being the one
 * the measuring CTA happened to run on.  Returns the number of SMs on the second side, or 0 (and an all-zero mask)
 * when the split is not known: switched off, the measurement could not run, or it did not show two halves.
 * No counterpart in the reference.
 */
int b200fp8_l2_sides(unsigned long long mask[3]);

/* "b200fp8 <version> sm_100a" */
const char* b200fp8_version(void);

#ifdef B200FP8_DIAGNOSTICS
/*
 * Only in a library built with -DB200FP8_DIAGNOSTICS (csrc/Makefile, target `diag`): the kernels
 * then honour the time-stamp and skip bits of the B200FP8_DEBUG environment variable.
 * b200fp8_debug_trace: DEVICE pointer of the time-stamp buffer, or NULL before the first traced launch.
 * b200fp8_debug_trace_copy: synchronises the device, copies the first `count` 64-bit words to `dst`,
 * optionally clears the buffer; returns the number of words copied.
 */
void* b200fp8_debug_trace(void);
int b200fp8_debug_trace_copy(long long* dst, int count, int clear);
#endif

#ifdef __cplusplus
}
#endif
#endif /* B200FP8_H */
