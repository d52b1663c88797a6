/*
 * sal_lutgemm.h — C ABI of the B200 (sm_100a) BCQ LUT-GEMV library.
 *
 * The library replaces the compiled `lutgemm` extension of ShiftAddLLM
 * (lut_gemm/lutgemm_cuda.cpp + lutgemm_cuda_kernel.cu + mv_fp16_bias.hpp).
 * Each compute entry point below names the reference function it stands in
 * for.  All pointers are DEVICE pointers owned by the caller unless stated
 * otherwise; the library keeps no state between calls and allocates nothing
 * on the compute path.  `stream` is a cudaStream_t passed as void* (NULL =
 * legacy default stream).  Every function returns SAL_OK (0) or a negative
 * SAL_E_* code; nothing is thrown and nothing is printed.
 *
 * Dimension names: K = in_features, N = out_features, M = rows (tokens),
 * q = bit planes (`nb`), num_groups as in the reference's argument lists.
 *
 * Common layouts (identical to the reference, mv_fp16_bias.hpp:52,86-90):
 *   bw     uint32 [K/32][q][N]   bit t of word kk = input feature 32*kk+t, set = +1
 *   x      fp16   [M][K]
 *   y      fp16   [M][N]
 *   bias   fp16   [N] or NULL
 *
 * Result: y = (flags & SAL_ACCUMULATE ? y : 0) + bias + sum_b alpha_b * (B_b^T x).
 * The reference kernels add into `output` (mv_fp16_bias.hpp:101); its callers
 * pre-load the bias there (lut_gemm/quant.py:46).  SAL_ACCUMULATE reproduces
 * that contract; without it the bias add is fused and y is overwritten.
 * Accumulation is fp32 and the split-K reduction order is fixed, so results
 * are deterministic (the reference accumulates in fp16 with atomics); the
 * accumulator outputs of SAL_OUT_FIXED_ATOMIC are deterministic too (integer sums).
 */
#ifndef SAL_LUTGEMM_H
#define SAL_LUTGEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAL_VERSION 100

/* status codes */
#define SAL_OK 0
#define SAL_E_NULL (-1)        /* a required pointer is NULL */
#define SAL_E_SHAPE (-2)       /* K % 32, group divisibility, q or M out of range ... */
#define SAL_E_ALIGN (-3)       /* pointer not 16-byte aligned */
#define SAL_E_WORKSPACE (-4)   /* workspace missing or too small */
#define SAL_E_LAUNCH (-5)      /* CUDA launch or runtime error */
#define SAL_E_UNSUPPORTED (-6) /* valid but not implemented for this shape */
#define SAL_E_DEVICE (-7)      /* no sm_100 device / wrong architecture */
#define SAL_E_TIMEOUT (-8)     /* a bounded device-side wait gave up (read back from the workspace) */

/* flags */
#define SAL_ACCUMULATE 1u  /* y += result (reference semantics) instead of y = bias + result */
#define SAL_PDL 2u         /* launch with programmatic dependent launch: the packed planes are
                              prefetched while the previous kernel of the stream drains */
#define SAL_FORCE_GENERIC 4u /* use the shape-agnostic kernel even where the tiled one applies */
#define SAL_OUT_FIXED_ATOMIC 8u /* y is INT64 [N], a fixed-point accumulator in units of 2**-32: bias + product is ADDED
                                  to it with 64-bit integer atomic adds (M = 1, tiled shapes only).  This is the
                                  reference's own output contract — its kernels atomicAdd into `output`
                                  (mv_fp16_bias.hpp:101) — carried out exactly: integer addition is associative, so the
                                  accumulated value does not depend on the order in which the thread blocks arrive and
                                  results are bit-identical from run to run.  Every partial sum is rounded once to
                                  2**-32 (2.3e-10); |y| must stay below 2**31.  No scratch and no split-K reduction
                                  tail.  The caller zeroes (or pre-loads) y; value = (double)y[n] * 2**-32. */
#define SAL_SWIGLU_FIXED 16u   /* with sal_problem.x_mul: x and x_mul are such INT64 accumulators (written with
                                  SAL_OUT_FIXED_ATOMIC), rounded to fp16 before silu(x) * x_mul is formed */

#define SAL_MAX_Q 8
#define SAL_MAX_M 64
#define SAL_MAX_GROUP 8 /* problems per grouped launch */
#define SAL_MAX_PEERS 8 /* GPUs taking part in a fused exchange */

int sal_version(void);
const char *sal_status_string(int status);

/* Text of the last CUDA runtime error seen by this thread inside the library
 * (what lies behind a SAL_E_LAUNCH). */
const char *sal_last_cuda_error(void);

/* Device check: SAL_OK when the current device is compute capability 10.x. */
int sal_device_ok(void);

/*
 * Scratch ("workspace") for the deterministic split-K reduction.  The caller
 * allocates `sal_workspace_bytes(M, N)` bytes of device memory once, zero-fills
 * it once (cudaMemset), and may reuse it for any later call whose M and N are
 * not larger.  Calls sharing one workspace must be ordered on one stream.
 * For a grouped launch pass the sum of N over the group.
 */
size_t sal_workspace_bytes(int M, int N);

/* Reads back (synchronously, on `stream`) and clears the device-side status
 * word of a workspace: SAL_OK or SAL_E_TIMEOUT. */
int sal_workspace_status(void *workspace, void *stream);

/*
 * Mode A ("row-wise groups"): alpha fp16 [num_groups][q][N], group = K/num_groups
 * consecutive input features.  Replaces lutgemm_compute_shift_scale
 * (lutgemm_cuda.cpp:43-52 -> lutgemm_cuda_kernel.cu:268-285 -> mv_fp16_bias.hpp:498-579,
 * 766-774).  The reference handles M = 1 only; here 1 <= M <= SAL_MAX_M.
 */
int sal_lutgemv_shift_scale(const void *bw, const void *alpha, const void *bias, const void *x, void *y,
                            int M, int K, int N, int q, int num_groups, unsigned flags,
                            void *workspace, size_t workspace_bytes, void *stream);

/*
 * sal_lutgemv_shift_scale without a caller-supplied workspace and without any allocation.
 * This entry has no counterpart in the reference.  It is for hosts that must not allocate device
 * memory once they are running: a serving process whose memory pool already owns the whole GPU, a
 * plugin called inside somebody else's stream capture (where cudaMalloc is illegal), an embedder
 * that was given a fixed budget at start-up.  The split-K scratch is a fixed array inside the
 * library image (about 4 MB per GPU that loads the library, held until the process exits), which
 * bounds the problem size: M * N <= 16384, otherwise SAL_E_WORKSPACE is returned and nothing runs.
 * Same arguments, results and flags as sal_lutgemv_shift_scale.
 *  - The first call on each device looks up the array's device address and, for shapes that use
 *    the tiled kernel, runs a one-off probe that synchronises the stream: make that first call
 *    outside any stream capture.
 *  - Every call uses the SAME array and first clears its arrival counters on `stream` (the status
 *    word is left for sal_static_status).
 *    Calls that can overlap on the GPU (different streams, or one stream with concurrent graph
 *    branches) race on it and give wrong results: keep them ordered, or use the workspace entry.
 *  - It calls no cudaMalloc/cudaFree and no allocating library routine.
 */
int sal_lutgemv_shift_scale_static(const void *bw, const void *alpha, const void *bias, const void *x, void *y,
                                   int M, int K, int N, int q, int num_groups, unsigned flags, void *stream);

/* Companion of sal_lutgemv_shift_scale_static (no counterpart in the reference either): reads back
 * (synchronously, on `stream`) and clears the device-side status word of the built-in scratch of the
 * current device — SAL_OK, SAL_E_TIMEOUT or SAL_E_UNSUPPORTED.  The word is sticky: calls of the
 * static entry leave it alone, so a status recorded by an earlier call is still there. */
int sal_static_status(void *stream);

/*
 * One alpha per (group, column), halved for each successive plane, plus an
 * offset term q_bias[g][n] * sum_{k in g} x[k].  alpha, q_bias fp16 [num_groups][N].
 * Replaces lutgemm_compute (lutgemm_cuda.cpp:88-98 -> lutgemm_cuda_kernel.cu:288-316
 * -> mv_fp16_bias.hpp:8-103, 726-734).
 */
int sal_lutgemv_compute(const void *bw, const void *alpha, const void *q_bias, const void *bias,
                        const void *x, void *y, int M, int K, int N, int q, int num_groups,
                        unsigned flags, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Mode B ("block"): one multiplier per block of 8 input features x (N/num_groups)
 * output features; alpha [K/8][q][num_groups].
 *   sal_lutgemm_block            alpha fp16                      replaces lutgemm_compute_block
 *       (lutgemm_cuda.cpp:54-63 -> lutgemm_cuda_kernel.cu:319-347 -> mv_fp16_bias.hpp:105-220)
 *   sal_lutgemm_block_shift      alpha uint16, three 3-bit exponents, multiplier
 *       2^(a&7)+2^((a>>3)&7)+2^((a>>6)&7)                        replaces lutgemm_compute_block_shift
 *       (lutgemm_cuda.cpp:65-74 -> lutgemm_cuda_kernel.cu:350-378 -> mv_fp16_bias.hpp:223-328)
 *   sal_lutgemm_block_shift_int8 alpha int8 [K/8][q][num_groups][3], multiplier sum of 2^s
 *       over the three shifts, -128 meaning "no term"            replaces lutgemm_compute_block_shiftInt8
 *       (lutgemm_cuda.cpp:76-85 -> lutgemm_cuda_kernel.cu:380-408 -> mv_fp16_bias.hpp:342-495);
 *       this is the call LutLinear.forward makes (lut_gemm/quant.py:50-51).
 * x fp16 [M][K], y fp16 [M][N], 1 <= M <= SAL_MAX_M.
 * Shapes with K % 256 == 0, N % 8 == 0, q <= 4 and N/num_groups = 16, 32, 64 (then num_groups % 4 == 0),
 * 128 or a multiple of 256 (int8: num_apot == 3) run on the TMA-ring kernel with a per-lookup multiplier
 * table in shared memory; all other shapes on the generic kernel (also selected by SAL_FORCE_GENERIC).
 */
int sal_lutgemm_block(const void *bw, const void *alpha, const void *bias, const void *x, void *y,
                      int M, int K, int N, int q, int num_groups, unsigned flags,
                      void *workspace, size_t workspace_bytes, void *stream);
int sal_lutgemm_block_shift(const void *bw, const void *alpha_u16, const void *bias, const void *x, void *y,
                            int M, int K, int N, int q, int num_groups, unsigned flags,
                            void *workspace, size_t workspace_bytes, void *stream);
int sal_lutgemm_block_shift_int8(const void *bw, const void *alpha_i8, const void *bias, const void *x, void *y,
                                 int M, int K, int N, int q, int num_groups, int num_apot, unsigned flags,
                                 void *workspace, size_t workspace_bytes, void *stream);

/*
 * Grouped mode-A launch: up to SAL_MAX_GROUP independent products in ONE kernel
 * (e.g. q/k/v of one decoder layer, or gate/up), so the weight stream does not
 * stop at problem boundaries.  No counterpart in the reference, which issues
 * one launch per linear layer (lut_gemm/quant.py:41-54).  `problems` is a HOST
 * array; it is copied into the launch parameters.
 */
typedef struct sal_problem {
    const void *bw;    /* uint32 [K/32][q][N] */
    const void *alpha; /* fp16 [num_groups][q][N] */
    const void *bias;  /* fp16 [N] or NULL */
    const void *x;     /* fp16 [M][K] */
    void *y;           /* fp16 [M][N] */
    int M, K, N, q, num_groups;
    const void *x_mul; /* optional fp16 [M][K] (NULL = unused): the activation becomes silu(x) * x_mul,
                          i.e. x = gate, x_mul = up of a SwiGLU block feeding this (down) projection */
} sal_problem;

int sal_lutgemv_grouped(const sal_problem *problems, int count, unsigned flags,
                        void *workspace, size_t workspace_bytes, void *stream);
/* All problems of a group share M and the activation form (x_mul or not).  Their plane counts q may
 * differ (layers of one block quantised to different widths, as the reference's per-layer mixed
 * precision does: model/opt.py:83-88,104-107): the group is then issued as one kernel per distinct q,
 * in the order the widths first appear. */

/*
 * Grouped launch with the all-gather of the output slices FUSED into the kernel (column-parallel
 * layers over the GPUs of one node).  No counterpart in the reference, which has no tensor
 * parallelism (model/opt.py:330-364 is a layer pipeline).  Every rank holds columns
 * [rank*N, (rank+1)*N) of each product (so sal_problem.N is the LOCAL width) and calls this with the
 * same shapes.  Besides writing problems[i].y, the CTA that finishes an output element stores it
 * (plain peer-to-peer stores over NVLink, no multicast) into EVERY peer buffer at element
 * gather_offsets[i] + rank*N + n, then adds 1 to counter `slot` of every rank's flag array
 * (system-scope release).  `*writers_out` receives the number of arrivals THIS rank contributes
 * per launch; with identical shapes on all ranks a rank has the complete gathered data once its
 * counter reaches world * writers — sal_exchange_wait does that wait.
 * peer_buffers / peer_flags: device pointers valid on this GPU for every rank's buffer (fp16) and
 * flag array (uint32), e.g. from CUDA IPC or torch symmetric memory; flags start at zero.
 * Use at least two slots in rotation (a slot is cleared by the wait that consumed it), and never make one
 * region of the gather buffers the target of two launches in a row: a peer that is one launch ahead may already
 * be storing launch L + 1's outputs into this rank's buffer while this rank still reads launch L's (it cannot be
 * further ahead: its launch L + 2 waits for this rank's arrival of L + 1, issued after this rank's reads of L).
 * The arrival is published by one release-add per peer after a CTA barrier.  M = 1 only.
 */
typedef struct sal_exchange {
    int world, rank, slot;
    void *peer_buffers[SAL_MAX_PEERS];
    void *peer_flags[SAL_MAX_PEERS];
    const long long *gather_offsets; /* HOST array, one element offset per problem */
} sal_exchange;

int sal_lutgemv_grouped_exchange(const sal_problem *problems, int count, unsigned flags,
                                 void *workspace, size_t workspace_bytes, const sal_exchange *exchange,
                                 int *writers_out, void *stream);

/*
 * Prepared launches: sal_lutgemv_grouped / sal_lutgemv_grouped_exchange split in two.  Preparing validates
 * the problems, plans the work split and encodes the tensor-map descriptors of the packed planes (driver
 * calls) ONCE; launching then only binds a scratch buffer and enqueues the kernel(s).  This is the form a
 * decoder uses: the same launches every token.  No counterpart in the reference (its launchers recompute
 * their grid on every call, mv_fp16_bias.hpp:581-645).
 *  - The pointers inside `problems` (and `exchange`, may be NULL) are remembered, not the memory behind
 *    them: the tensors must stay where they are while the handle is used.
 *  - A handle belongs to the device that was current when it was prepared.
 *  - `workspace` as for sal_lutgemv_grouped, at least sal_prepared_workspace_bytes() bytes.
 *  - `slot`: counter slot of a fused-exchange launch (ignored without exchange; < 0 keeps the slot given
 *    at preparation).  sal_prepared_writers: arrivals this rank contributes per launch (0 without exchange).
 */
typedef struct sal_prepared sal_prepared;
int sal_prepare_grouped(const sal_problem *problems, int count, unsigned flags, const sal_exchange *exchange,
                        sal_prepared **out);
size_t sal_prepared_workspace_bytes(const sal_prepared *prepared);
int sal_prepared_writers(const sal_prepared *prepared);
int sal_launch_prepared(const sal_prepared *prepared, void *workspace, size_t workspace_bytes, int slot, void *stream);
/* `count` prepared launches enqueued one after the other by ONE call (a decoder block, a whole token): the host
 * cost per launch is then the CUDA launch itself.  `slots` (may be NULL) gives the counter slot of each launch. */
int sal_launch_prepared_sequence(const sal_prepared *const *prepared, int count, const int *slots, void *workspace,
                                 size_t workspace_bytes, void *stream);
void sal_destroy_prepared(sal_prepared *prepared);

/* Enqueues a one-thread kernel that waits (bounded, about one second; SAL_E_TIMEOUT is recorded
 * in the workspace status word if it gives up) until counter `slot` of this rank's flag array
 * reaches `expected`, then clears it.  `workspace` may be NULL (no status reporting). */
int sal_exchange_wait(void *local_flags, int slot, unsigned expected, void *workspace, void *stream);

/* Introspection for tests and the benchmark: which kernel a mode-A call would
 * use (1 = tiled TMA kernel, 0 = generic) and its launch geometry. */
typedef struct sal_plan_info {
    int tiled;
    int ctas;
    int ranges;      /* column ranges */
    int splits;      /* K splits */
    int stages;
    int smem_bytes;
} sal_plan_info;
int sal_plan_shift_scale(int M, int K, int N, int q, int num_groups, sal_plan_info *out);

#ifdef SAL_MEASURE
/* Measurement hook, process-wide; exists only in libraries built with -DSAL_MEASURE (the product
 * build has neither this symbol nor the switches it sets).  Keys: "stages" caps the
 * depth of the shared-memory ring of the tiled kernel (0 = as deep as fits);
 * "budget_pct" scales the number of SMs the planner sizes its grid for
 * (100 = one CTA per SM, 200 = two, 0 = automatic); "full_sm" lets a CTA use a
 * whole SM's shared memory (one CTA per SM, deeper ring); "abs" 0/1 forces the table
 * addressing variant; "ablate" bit0/1/2 skips alpha loads / table builds /
 * lookups, bit3/4 the multiplier stores / per-tile barrier of the block mode
 * (results are then meaningless; used to time the parts); "force_per" and
 * "force_splits" override the planner's column tiles per CTA and K splits. */
int sal_debug_set(const char *key, int value);
/* Measurement builds only: copies the per-CTA cycle counters of the last tiled launches to `host` (at most 64 KB):
 * 8 x uint64 per (CTA, consumer warp 0 | 7) for the first 512 CTAs — cycles at the dependency wait, cycles waiting
 * for ring data, cycles in table builds, cycles of the main loop, units, K blocks, SM id, problem index. */
int sal_debug_read(void *host, size_t bytes);
#endif

#ifdef __cplusplus
}
#endif
#endif /* SAL_LUTGEMM_H */
