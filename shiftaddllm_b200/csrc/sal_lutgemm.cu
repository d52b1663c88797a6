// BCQ LUT-GEMV for NVIDIA B200 (sm_100a): kernels and the C ABI declared in
// include/sal_lutgemm.h.
//
// y[n] = sum_g sum_b alpha[g][b][n] * sum_{chunk c in g} LUT_c[ byte_c(bw[.][b][n]) ]
//
// where LUT_c is the 256-entry table of signed partial sums of the eight
// activations of chunk c.  The packed bit planes are streamed from HBM exactly
// once and never dequantised.
//
// Tiled kernel (M = 1, mode A), per CTA:
//   * one producer thread issues tiled TMA copies (cp.async.bulk.tensor.3d through a
//     tensor map of the packed planes seen as [K/32][q][N], completion on mbarrier
//     transaction counts) of [8 words][planes][256 columns] boxes into a shared-memory
//     ring: all planes of a (K block, column tile) unit in one slot up to q = 3 (16 or 24 KB,
//     three or two slots), two planes per slot for q = 4.  The copies do not depend on the activations, so
//     under programmatic dependent launch they are issued before
//     griddepcontrol.wait and overlap the previous kernel's tail.  A CTA uses
//     at most half of an SM's shared memory, so the CTAs of two consecutive
//     kernels are co-resident: one computes while the next one's weights land;
//   * the alpha scales are read with plain loads, one tile ahead, into registers;
//   * NCW consumer warps build the tables of one 256-feature K block in shared
//     memory, "bank striped": entry e of chunk c sits at byte e*256 + 4*c (+128
//     for odd K blocks, which double-buffers the table), so chunk c only ever
//     touches bank c;
//   * lookups are skewed so that at every step the 32 lanes of a warp address
//     32 different chunks, i.e. 32 different banks: lane l owns output column
//     l of its strip and walks the 8 words of the K block in a lane-dependent
//     rotation.  The shared-memory address of a lookup is produced by a single
//     byte-permute (byte -> bits 8..15, lane/step constant -> bits 0..7);
//   * fp32 accumulation; K splits are reduced through a global scratch buffer
//     by the last CTA to arrive (fixed summation order, so deterministic).
//
// Every wait on an mbarrier is bounded; on expiry the kernel records
// SAL_E_TIMEOUT in the workspace header and carries on to its exit.

#include <cuda.h>
#include <cuda_fp16.h>
#include <mutex>
#include <new>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "sal_lutgemm.h"

namespace {

// ------------------------------------------------------------------------------------------
// constants shared by host and device
// ------------------------------------------------------------------------------------------
constexpr int KB_WORDS = 8;                  // 32-bit words of K per K block
constexpr int KB_FEATS = KB_WORDS * 32;      // 256 input features per K block
constexpr int LUT_ROW_BYTES = 256;           // one table entry index = one 256-byte row
constexpr int LUT_BYTES = 256 * LUT_ROW_BYTES;  // 64 KB: two K blocks' tables, interleaved by half rows
constexpr int MAX_SUB = 8;                   // column sub-tiles per CTA (accumulators per lane)
constexpr int MAX_SPLIT = 64;                // K splits supported by the workspace layout
constexpr int WS_HEADER_BYTES = 256;
constexpr int WS_COUNTER_BYTES = 16384 - WS_HEADER_BYTES;
constexpr int WS_MAX_COUNTERS = WS_COUNTER_BYTES / 4;
constexpr size_t WS_PARTIAL_OFFSET = 16384;
constexpr int BOX_COLS = 256;             // columns of one TMA box (the limit of a tensor-map box dimension)
constexpr int ACT_BYTES = KB_FEATS * 2;   // one K block of fp16 activations, staged by the SwiGLU variants (M = 1)

enum AlphaKind { A_ROW_F16 = 0, A_ROW_HALVING = 1, B_F16 = 2, B_U16 = 3, B_I8 = 4 };

struct TileProblem {
    const uint32_t *bw;
    const __half *alpha;
    const __half *bias;
    const __half *x;
    const __half *x_mul;  // optional: the activation is silu(x) * x_mul (SwiGLU feeding a down projection)
    __half *y;
    float *partials;     // [splits][N]
    unsigned *counters;  // [ranges]
    int K, N, M;
    int g;               // group size along K, multiple of 128
    int kblocks;         // K / 256
    int nsub_total;      // ceil(N / CW)
    int nsub_per_range;  // column tiles per range (the last range may be narrower)
    int ranges;
    int splits;          // CTAs per full-width range
    int splits_last;     // CTAs of the last range
    int cta_begin;
    // block mode (one multiplier per 8 input features x `blk_gs` output columns, alpha [K/8][q][N/blk_gs]):
    int blk_kind;     // 0 = off (alpha per K group and column), else the AlphaKind of the multipliers
    int blk_gs;       // columns per group: 16, 32, 64, 128 or a multiple of 256
    int blk_ngroups;  // N / blk_gs
    int blk_apot;     // int8 encoding: exponents per multiplier (<= 4)
    long long gather_off;  // fused exchange: element offset of this problem's [world][N] block in the peer buffers
};

// Fused all-gather of the output slices (column-parallel layers): every finished y element is
// also stored into the same place of every peer's buffer, then one counter per peer is bumped.
struct ExchangeParams {
    int world;   // 0/1: off
    int rank;
    int slot;    // which counter of the flag arrays this launch signals
    int pad_;
    __half *base[SAL_MAX_PEERS];
    unsigned *flags[SAL_MAX_PEERS];
};

struct TileParams {
    // One tiled-TMA descriptor per problem: the packed planes seen as a 3-D uint32 tensor
    // [K/32 words][q planes][N columns], box = [8 words][PPS planes][256 columns] = one ring slot.
    alignas(64) CUtensorMap tmap[SAL_MAX_GROUP];
    TileProblem p[SAL_MAX_GROUP];
    int count;
    int stages;
    int accumulate;
    int ablate;  // measurement builds (-DSAL_MEASURE) only: bit0 skip alpha loads, bit1 skip table builds, bit2 skip
                 // lookups; block mode: bit3 skip the multiplier decode + stores, bit4 skip the per-tile barrier
    int *status;
    ExchangeParams ex;
};

// Parts of the kernel can be switched off to time the others; only in measurement builds, so that
// the product's hot loop carries no such test and its results cannot be made meaningless.
#ifdef SAL_MEASURE
#define SAL_ABLATED(P, bits) (((P).ablate & (bits)) != 0)
#else
#define SAL_ABLATED(P, bits) false
#endif

// ------------------------------------------------------------------------------------------
// PTX helpers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after about one second and reports it through `status`.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int *status) {
    if (mbar_try_wait(bar, parity)) return;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return;
        if (global_timer_ns() - t0 > 1000000000ull) {
            if (status) atomicExch(status, SAL_E_TIMEOUT);
            return;
        }
    }
}
// prmt.b32, generic mode: selector nibble bits 0-2 pick one of the eight source bytes,
// bit 3 replaces the byte by eight copies of its sign bit.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
    return d;
}
// Fixed-point accumulators (SAL_OUT_FIXED_ATOMIC): signed 64-bit integers counting units of 2**-32.  Integer
// addition is associative, so the value left by any number of atomic adds does not depend on their order.
constexpr float SAL_FIXED_ONE = 4294967296.f;            // 2**32
constexpr float SAL_FIXED_INV = 2.3283064365386963e-10f; // 2**-32
__device__ __forceinline__ unsigned long long to_fixed(float v) { return (unsigned long long)__float2ll_rn(v * SAL_FIXED_ONE); }
__device__ __forceinline__ float from_fixed(long long v) { return __ll2float_rn(v) * SAL_FIXED_INV; }

// Read-once data (alpha): not kept in L1, so that it does not push out the few lines that are reused (the prefetched
// activations of the next K block, the accumulators of the two-row kernel).
__device__ __forceinline__ __half ldg_stream_f16(const __half *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __ushort_as_half(v);
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
template <int IMM>
__device__ __forceinline__ float lds_f32_imm(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(IMM));
    return v;
}
template <int IMM>
__device__ __forceinline__ uint32_t lds_u32_imm(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Tiled TMA load of one 3-D box (no multicast).  x is the innermost (column) coordinate in
// elements and must keep x * 4 bytes a multiple of 16; y is the plane, z the first 32-bit word of K.
__device__ __forceinline__ void tma_tile_3d_g2s(uint32_t dst, const CUtensorMap *tmap, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void consumer_barrier(int nthreads) {
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------------------------
// tiled kernel
// ------------------------------------------------------------------------------------------
template <int Q, int NCW>
struct TileCfg {
    static constexpr int CW = NCW * 32;             // columns per stage
    static constexpr int PPS = (Q == 4 ? 2 : Q);    // planes per ring slot: all of them up to q = 3, two slots per unit for q = 4
    static constexpr int SLOTS = Q / PPS;           // ring slots per (K block, column tile) unit
    static constexpr int W_ROWS = KB_WORDS * PPS;   // weight rows per slot: [8 words][PPS planes]
    static constexpr int STAGE_BYTES = W_ROWS * CW * 4;
    static constexpr int THREADS = (NCW + 1) * 32;   // consumer warps + the copy warp
};

// Builds the 32 tables of one K block.  Lane = chunk; a warp handles groups of
// eight consecutive entries (entry >> 3 = hgrp).  Bank of every store = lane.
// Builds the 32 tables of one K block.  Lane = chunk; a warp handles groups of eight consecutive
// entries (entry >> 3 = hg).  Bank of every store = lane.  ROWS = 1: fp32 entries of activation
// row x0.  ROWS = 2: half2 entries, low half = row x0, high half = row x1 (sums are formed in
// fp32 and rounded once).
template <int NCW, int ROWS>
__device__ __forceinline__ void store_tables(const float (&xf)[ROWS][8], uint32_t lut_half, int warp, int lane);

template <int NCW, int ROWS, int SWIGLU>
__device__ __forceinline__ void build_tables_impl(const __half *__restrict__ x0, const __half *__restrict__ x1,
                                                  const __half *__restrict__ m0, const __half *__restrict__ m1,
                                                  uint32_t lut_half, int warp, int lane) {
    float xf[ROWS][8];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        if (SWIGLU == 4) {
            // the K block's activations were formed once per CTA and staged in shared memory as fp16 (x0 = their
            // generic address); lane = chunk takes its eight
            const uint4 raw = *(reinterpret_cast<const uint4 *>(x0) + lane);
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                xf[r][2 * i] = f.x;
                xf[r][2 * i + 1] = f.y;
            }
            continue;
        }
        if (SWIGLU == 2) {
            // gate and up are the fixed-point accumulators two earlier products added into (plain loads: they were
            // written by atomics of the previous kernels, not constant data)
            const longlong2 *gp = reinterpret_cast<const longlong2 *>(r == 0 ? x0 : x1) + 4 * lane;
            const longlong2 *up = reinterpret_cast<const longlong2 *>(r == 0 ? m0 : m1) + 4 * lane;
            long long g[8], u[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const longlong2 gv = gp[i], uv = up[i];
                g[2 * i] = gv.x, g[2 * i + 1] = gv.y, u[2 * i] = uv.x, u[2 * i + 1] = uv.y;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float gi = __half2float(__float2half_rn(from_fixed(g[i])));   // the two-step path rounds gate and up to fp16 first
                const float sg = __half2float(__float2half_rn(gi / (1.f + __expf(-gi))));
                xf[r][i] = __half2float(__float2half_rn(sg * __half2float(__float2half_rn(from_fixed(u[i])))));
            }
            continue;
        }
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(r == 0 ? x0 : x1) + lane);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            xf[r][2 * i] = f.x;
            xf[r][2 * i + 1] = f.y;
        }
        if (SWIGLU == 1) {
            // fused SwiGLU: the activation is silu(gate) * up, rounded to fp16 after each step exactly as
            // the separate element-wise kernel (and torch's fp16 ops) would produce it
            const uint4 mraw = __ldg(reinterpret_cast<const uint4 *>(r == 0 ? m0 : m1) + lane);
            const __half *mh = reinterpret_cast<const __half *>(&mraw);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float g = xf[r][i];
                const float sg = __half2float(__float2half_rn(g / (1.f + __expf(-g))));
                xf[r][i] = __half2float(__float2half_rn(sg * __half2float(mh[i])));
            }
        }
    }
    store_tables<NCW, ROWS>(xf, lut_half, warp, lane);
}

template <int NCW, int ROWS>
__device__ __forceinline__ void store_tables(const float (&xf)[ROWS][8], uint32_t lut_half, int warp, int lane) {
    float low[ROWS][8];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i)
            low[r][i] = ((i & 1) ? xf[r][0] : -xf[r][0]) + ((i & 2) ? xf[r][1] : -xf[r][1]) + ((i & 4) ? xf[r][2] : -xf[r][2]);
    const uint32_t dst = lut_half + 4u * lane;
#pragma unroll 1
    for (int hg = warp; hg < 32; hg += NCW) {
        float hi[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            hi[r] = ((hg & 1) ? xf[r][3] : -xf[r][3]) + ((hg & 2) ? xf[r][4] : -xf[r][4]) + ((hg & 4) ? xf[r][5] : -xf[r][5]) +
                    ((hg & 8) ? xf[r][6] : -xf[r][6]) + ((hg & 16) ? xf[r][7] : -xf[r][7]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t a = dst + (uint32_t)(hg * 8 + i) * LUT_ROW_BYTES;
            if (ROWS == 1) {
                sts_f32(a, hi[0] + low[0][i]);
            } else {
                const __half2 e = __floats2half2_rn(hi[0] + low[0][i], hi[ROWS - 1] + low[ROWS - 1][i]);
                sts_f32(a, __uint_as_float(*reinterpret_cast<const uint32_t *>(&e)));
            }
        }
    }
}

// Fused exchange, producer side.  A finished output element is stored into every peer's gather
// buffer with a plain peer-to-peer store (NVLink): slice `rank` of the problem's [world][N] block.
__device__ __forceinline__ void push_to_peers(const ExchangeParams &ex, long long gather_off, int N, int n, __half v) {
    const long long off = gather_off + (long long)ex.rank * N + n;
    for (int t = 0; t < ex.world; ++t) ex.base[t][off] = v;  // includes this rank's own gather buffer
}
// After all threads of a writer CTA pushed their elements: one CTA barrier, then ONE thread per peer publishes
// them with a system-scope release add on that peer's counter of this launch (and on this rank's own).  The
// release is cumulative: the pushes of the other threads happen before it through the barrier, so an acquire
// load that sees the count also sees the data.  (A __threadfence_system() in each of the 256 threads before
// the barrier, as an earlier version had, made every thread wait for the NVLink round trip of its own
// stores.)  One arrival per writer CTA.
__device__ __forceinline__ void signal_peers(const ExchangeParams &ex, int tid, int nthreads) {
    consumer_barrier(nthreads);
    if (tid < ex.world) {
        unsigned *flag = ex.flags[tid] + ex.slot;
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
    }
}

// Fused exchange, consumer side: waits (bounded, ~1 s) until `expected` writer CTAs of all ranks
// have signalled counter `flag`, then clears it for the next use.  Launched between the producing
// launch and whatever reads the gathered data on this rank.
__global__ void exchange_wait_kernel(unsigned *flag, unsigned expected, int *status) {
    // Let the next kernel of the stream start right away: it prefetches its weights while this
    // thread waits for the peers, and only proceeds past its own griddepcontrol.wait once this
    // kernel has finished.  Polling before the producing launch has finished is harmless.
    pdl_launch_dependents();
    if (threadIdx.x != 0) return;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= expected) break;
        if (global_timer_ns() - t0 > 1000000000ull) {
            if (status) atomicExch(status, SAL_E_TIMEOUT);
            break;
        }
    }
    *flag = 0u;
}

// Measurement builds keep cycle counters of the consumer warps 0 and 7 of every CTA (first 512 CTAs, row group 0):
// [cycles at the dependency wait, cycles waiting for ring data, cycles in table builds incl. their barrier, cycles
// of the main loop, units, K blocks, SM id, problem].  sal_debug_read copies them out.  In the product build the
// macros vanish.
#ifdef SAL_MEASURE
__device__ unsigned long long g_cta_timers[1024 * 8];
#define SAL_CYCLES() clock64()
#else
#define SAL_CYCLES() 0ll
#endif

// Shared-window address at which the dynamic shared memory of a kernel without static
// shared memory starts on sm_100 (the first KB of every CTA's allocation is reserved by the
// driver).  The ABS variant of the kernel bakes the table address into the immediate field of
// its lookups; it verifies the assumption at run time and reports SAL_E_UNSUPPORTED through
// the status word instead of computing if it does not hold.
constexpr uint32_t SMEM_DYNAMIC_BASE = 1024;

// ROWS = 1: the M = 1 kernel.  ROWS = 2: small-batch variant, blockIdx.y = pair of activation
// rows; the same weight tile serves both rows through half2 table entries.  SWIGLU: the activation
// is silu(x) * x_mul, formed while the tables are built (a separate instantiation, so that the
// extra registers of that prologue do not weigh on the ordinary kernel).  EXCH: the fused all-gather
// epilogue (peer stores + counters), likewise its own instantiation.  SWIGLU = 2: gate and up are such fixed-point accumulators.
// ATOMIC: y is a 64-bit fixed-point accumulator [N] (units of 2**-32); every CTA adds its partial sums with
// integer atomics (no scratch, no reduction tail; integer sums do not depend on the order of arrival).
// BLK: block mode.  Every lookup has its own multiplier alpha[chunk][plane][column / gs].  The multipliers
// of a tile (32 chunks x Q planes x up to 16 column groups) are fetched one tile ahead, decoded to fp32
// and parked in the upper 128 bytes of the table rows (this mode keeps ONE set of tables, in the lower
// halves): row (buffer * Q + plane) * 16 + group, chunk c of group gi at byte 128 + 4 * (c ^ gi), which
// makes both the decode stores and the skewed reads conflict-free.  ROWS = 1, blockIdx.y = activation row.
template <int Q, int NCW, bool ABS, int ROWS, int SWIGLU, bool EXCH, bool ATOMIC, bool BLK>
__global__ void __launch_bounds__(TileCfg<Q, NCW>::THREADS, (NCW <= 8 ? 2 : 1))
    lutgemv_tiled_kernel(const __grid_constant__ TileParams P) {
    static_assert(!BLK || (ROWS == 1 && SWIGLU == 0 && !EXCH && !ATOMIC && Q <= 8), "block mode: plain M-row kernel only");
    using C = TileCfg<Q, NCW>;
    constexpr int CW = C::CW;
    extern __shared__ __align__(128) unsigned char smem[];

    unsigned char *stage_base = smem + LUT_BYTES;
    const uint32_t lut_s = smem_u32(smem);
    const uint32_t stage_s = smem_u32(stage_base);
    const int stages = P.stages;
    uint64_t *bars = reinterpret_cast<uint64_t *>(stage_base + (size_t)stages * C::STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + stages);
    volatile int &s_last = *reinterpret_cast<volatile int *>(bars + 2 * stages);
    __half *act_s = reinterpret_cast<__half *>(bars + 2 * stages + 2);   // ACT_BYTES, 16-byte aligned

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (ABS && lut_s != SMEM_DYNAMIC_BASE) {  // uniform over the grid: everybody leaves
        if (tid == 0 && P.status) atomicExch(P.status, SAL_E_UNSUPPORTED);
        return;
    }

    // which problem / column range / K split / activation rows is this CTA
    int pi = 0;
#pragma unroll 1
    for (int i = 1; i < P.count; ++i)
        if ((int)blockIdx.x >= P.p[i].cta_begin) pi = i;
    const TileProblem &pr = P.p[pi];
    // Work of a column range = its (K block, column tile) units in K-block-major order; the range's CTAs
    // take equal contiguous runs of that sequence, so a CTA may start and end in the middle of a K block.
    const int local = blockIdx.x - pr.cta_begin;
    const int full_ctas = (pr.ranges - 1) * pr.splits;
    const bool in_last = local >= full_ctas;
    const int range = in_last ? pr.ranges - 1 : local / pr.splits;
    const int split = in_last ? local - full_ctas : local % pr.splits;
    const int S = in_last ? pr.splits_last : pr.splits;  // CTAs sharing this range
    const int N = pr.N;
    const int row0 = (int)blockIdx.y * ROWS;
    const int rows_here = min(ROWS, pr.M - row0);
    const int sub_begin = range * pr.nsub_per_range;
    const int nsub = min(pr.nsub_per_range, pr.nsub_total - sub_begin);
    const int units = nsub * pr.kblocks;
    const int u_begin = (int)(((long long)split * units) / S);
    const int u_end = (int)(((long long)(split + 1) * units) / S);   // > u_begin: the planner keeps S <= units
    const int kb_begin = u_begin / nsub, t_first = u_begin % nsub;   // first K block and its first tile
    const int kb_last = (u_end - 1) / nsub, t_last = (u_end - 1) % nsub;
    const int kb_end = kb_last + 1;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, NCW);
        }
        fence_barrier_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == NCW) {
        // ------------------------------ producer warp ------------------------------
        int st = 0;
        uint32_t phase = 0;  // parity of the consumers' release being waited for (previous use of the stage)
        bool first_round = true;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            const int s_lo = kb == kb_begin ? t_first : 0, s_hi = kb == kb_last ? t_last + 1 : nsub;
            for (int sub = s_lo; sub < s_hi; ++sub) {
                const int n0 = (sub_begin + sub) * CW;
#pragma unroll 1
                for (int b = 0; b < Q; b += C::PPS) {   // one slot per PPS planes
                    if (!first_round) mbar_wait(empty0 + 8 * st, phase, P.status);
                    const uint32_t full = full0 + 8 * st;
                    if (lane == 0) {
                        // columns past N are zero-filled by the TMA unit and still counted
                        mbar_expect_tx(full, (uint32_t)C::STAGE_BYTES);
#pragma unroll
                        for (int bx = 0; bx < CW / BOX_COLS; ++bx)
                            tma_tile_3d_g2s(stage_s + (uint32_t)st * C::STAGE_BYTES + (uint32_t)bx * (C::W_ROWS * BOX_COLS * 4),
                                            &P.tmap[pi], n0 + bx * BOX_COLS, b, kb * KB_WORDS, full);
                    }
                    __syncwarp();
                    if (++st == stages) {
                        st = 0;
                        if (first_round) first_round = false;
                        else phase ^= 1u;
                    }
                }
            }
        }
        return;
    }

    const __half *xrow0 = pr.x + (size_t)row0 * pr.K;
    const __half *xrow1 = pr.x + (size_t)(row0 + (rows_here > 1 ? 1 : 0)) * pr.K;  // odd M: the last pair repeats its row
    // Tables of K block `kb` into table half `half`, by `nwarps` warps of which this is number `w`.
    auto build_block = [&](int kb, int half, int w, auto nwarps_tag) {
        constexpr int NW = decltype(nwarps_tag)::value;
        const size_t ko = (size_t)kb * KB_FEATS;
        if (SWIGLU != 0 && ROWS == 1) {
            // silu(gate) * up of the K block's 256 features, ONE per consumer thread, staged as fp16; the warps then build
            // from the staged values.  (Each warp forming all 256 itself, as the plain-activation path does with its
            // single 16-byte load, costs eight times the conversions, exponentials and divisions.)  Rounded step by
            // step exactly as the separate element-wise kernel (and torch's fp16 ops) would round.
            float gi, ui;
            if (SWIGLU == 2) {   // 64-bit fixed-point accumulators written by the atomics of earlier kernels: plain loads
                const long long *gp = reinterpret_cast<const long long *>(pr.x) + ko, *up = reinterpret_cast<const long long *>(pr.x_mul) + ko;
                gi = __half2float(__float2half_rn(from_fixed(gp[tid])));
                ui = __half2float(__float2half_rn(from_fixed(up[tid])));
            } else {
                gi = __half2float(pr.x[ko + tid]);
                ui = __half2float(pr.x_mul[ko + tid]);
            }
            const float sg = __half2float(__float2half_rn(gi / (1.f + __expf(-gi))));
            act_s[tid] = __float2half_rn(sg * ui);
            consumer_barrier(NCW * 32);
            build_tables_impl<NW, 1, 4>(act_s, nullptr, nullptr, nullptr, lut_s + half * 128, w, lane);
            return;
        }
        if (SWIGLU == 1 && ROWS == 2) {
            // the same for a pair of rows, one after the other through the one staging buffer
            float xf[2][8];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const __half *grow = (r == 0 ? xrow0 : xrow1) + ko;
                const __half *urow = pr.x_mul + (grow - pr.x);   // x_mul row = x_mul + (the same element offset the x row has)
                const float gi = __half2float(grow[tid]);
                const float sg = __half2float(__float2half_rn(gi / (1.f + __expf(-gi))));
                act_s[tid] = __float2half_rn(sg * __half2float(urow[tid]));
                consumer_barrier(NCW * 32);
                const uint4 raw = *(reinterpret_cast<const uint4 *>(act_s) + lane);
                const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(h[i]);
                    xf[r][2 * i] = f.x;
                    xf[r][2 * i + 1] = f.y;
                }
                if (r == 0) consumer_barrier(NCW * 32);   // everybody has its eight before the second row overwrites them
            }
            store_tables<NW, 2>(xf, lut_s + half * 128, w, lane);
            return;
        }
        if (SWIGLU == 2) {   // 64-bit fixed-point operands: same element offsets, four times the bytes (pointers are carried as __half*)
            const __half *g32 = pr.x + 4 * ((xrow0 - pr.x) + ko);
            const __half *u32 = pr.x_mul + 4 * ((xrow0 - pr.x) + ko);
            build_tables_impl<NW, ROWS, SWIGLU>(g32, g32, u32, u32, lut_s + half * 128, w, lane);
        } else {
            // x_mul row = x_mul + (the same element offset the x row has)
            const __half *m0 = SWIGLU ? pr.x_mul + (xrow0 - pr.x) + ko : nullptr;
            const __half *m1 = SWIGLU ? pr.x_mul + (xrow1 - pr.x) + ko : nullptr;
            build_tables_impl<NW, ROWS, SWIGLU>(xrow0 + ko, xrow1 + ko, m0, m1, lut_s + half * 128, w, lane);
        }
    };
    // -------------------------------- consumer warps --------------------------------
    const int col = warp * 32 + lane;
    const int hw = lane >> 4;
    const int rot = (lane >> 2) & 3;
    const int s4 = lane & 3;
    // Lookup address = one byte-permute of (weight word, packed constants):
    //   byte 0 <- 4*chunk (the bank), taken from byte t of cpack
    //   byte 1 <- the weight byte (table entry index; one entry = one 256-byte row)
    //   bytes 2,3 <- sign replication of a constant < 128, i.e. zero.
    unsigned sel[4];
    unsigned cpack[2][4];
    unsigned wrow[2][4];
#pragma unroll
    for (int t = 0; t < 4; ++t)
        sel[t] = (unsigned)(4 + t) | (unsigned)(((t + s4) & 3) << 4) | (unsigned)((8 | (4 + t)) << 8) |
                 (unsigned)((8 | (4 + t)) << 12);
#pragma unroll
    for (int hp = 0; hp < 2; ++hp)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int wi = 4 * (hp ^ hw) + ((j + rot) & 3);
            wrow[hp][j] = stage_s + (unsigned)(((col / BOX_COLS) * (C::W_ROWS * BOX_COLS) + wi * C::PPS * BOX_COLS + (col % BOX_COLS)) * 4);
            unsigned pk = 0;
#pragma unroll
            for (int t = 0; t < 4; ++t) pk |= (unsigned)(16 * wi + 4 * ((t + s4) & 3)) << (8 * t);
            cpack[hp][j] = pk;
        }
    // block mode: the same chunk offsets with the lane's group folded in, and the row of the lane's group
    unsigned mpack[BLK ? 2 : 1][BLK ? 4 : 1];
    uint32_t mrow = 0;
    int blk_gt = 1, blk_gshift = 0;  // column groups per tile and its log2
    if constexpr (BLK) {
        if (pr.blk_gs < BOX_COLS) {
            blk_gt = BOX_COLS / pr.blk_gs;
            blk_gshift = 31 - __clz(blk_gt);
        }
        const unsigned grp = pr.blk_gs < BOX_COLS ? (unsigned)(col / pr.blk_gs) : 0u;
        mrow = grp * (unsigned)LUT_ROW_BYTES;
#pragma unroll
        for (int hp = 0; hp < 2; ++hp)
#pragma unroll
            for (int j = 0; j < 4; ++j) mpack[hp][j] = cpack[hp][j] ^ (0x01010101u * (4u * grp));
    }

    float acc[ROWS][MAX_SUB];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int i = 0; i < MAX_SUB; ++i) acc[r][i] = 0.f;

    // alpha for one tile: the (up to) two groups of the K block x Q planes, fetched one tile ahead
    // with loads whose address is "per-lane column pointer + warp-uniform offset".  Columns past
    // N are clamped to N-1 (their results are never stored), so the loads need no predicate.
    const int two_groups = (pr.g == 128) ? 1 : 0;
    const int gdiv = pr.g / 128;  // 128-feature units per group
    auto load_alpha = [&](int kb, int sub, __half(&dst)[2][Q]) {
        const int n = min((sub_begin + sub) * CW + col, N - 1);
        const int g0 = two_groups ? 2 * kb : (2 * kb) / gdiv;
        const __half *p0 = pr.alpha + n;
        const size_t off0 = (size_t)g0 * Q * (size_t)N;
        const size_t off1 = off0 + (two_groups ? (size_t)Q * (size_t)N : 0);
#pragma unroll
        for (int b = 0; b < Q; ++b) {
            dst[0][b] = ldg_stream_f16(p0 + off0 + (size_t)b * N);
            dst[1][b] = ldg_stream_f16(p0 + off1 + (size_t)b * N);
        }
    };
    __half a_next[2][Q];
    if (!BLK && kb_begin < kb_end && !SAL_ABLATED(P, 1)) load_alpha(kb_begin, t_first, a_next);  // constants: legal before the dependency wait
    else {
#pragma unroll
        for (int b = 0; b < Q; ++b) a_next[0][b] = a_next[1][b] = __float2half(0.f);
    }
    // block mode, multipliers of one tile (32 chunks x Q planes x `blk_gt` column groups), fetched by the
    // 256 consumer threads.  16/8/4 groups per tile: item e = tid + 256 i is FOUR consecutive groups
    // (one 8- or 12-byte run of alpha) of one (chunk, plane); 1 or 2 groups per tile: item = one value.
    // The chunk bits of an item are arranged so that the 32 stores of a warp hit 32 different banks.
    constexpr int NVI = BLK ? (Q + 1) / 2 : 1;   // items per thread
    constexpr int NVW = BLK ? 3 : 1;             // 32-bit words per item (12 bytes of int8 x 3, 8 bytes of 16-bit)
    uint32_t raw_next[NVI][NVW];
    const bool blk_quads = blk_gt >= 4;
    auto item_coords = [&](int e, int &gi, int &c, int &b) {
        if (blk_quads) {
            const int qmask = (blk_gt >> 2) - 1, cb = e >> (blk_gshift - 2);
            gi = (e & qmask) << 2;
            c = (cb & 3) | (((cb >> 3) & 3) << 2) | (((cb >> 2) & 1) << 4);
            b = cb >> 5;
        } else {
            const int idx = e >> blk_gshift;
            gi = e & (blk_gt - 1);
            c = ((idx & 1) << 4) | ((idx >> 1) & 15);
            b = idx >> 5;
        }
    };
    auto load_block_alpha = [&](int kb, int sub, uint32_t(&dst)[NVI][NVW]) {
        const int g0 = ((sub_begin + sub) * CW) / pr.blk_gs;
#pragma unroll
        for (int i = 0; i < NVI; ++i) {
            int gi, c, b;
            item_coords(tid + 256 * i, gi, c, b);
            dst[i][0] = dst[i][1] = dst[i][2] = 0u;
            if (b < Q) {
                // groups past the last one belong to columns past N, whose results are never stored
                const int gq = min(g0 + gi, pr.blk_ngroups - (blk_quads ? 4 : 1));
                const size_t a = ((size_t)(kb * 32 + c) * Q + b) * pr.blk_ngroups + gq;
                if (blk_quads) {
                    if (pr.blk_kind == B_I8) {
                        const uint32_t *ap = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(pr.alpha) + a * 3);
                        dst[i][0] = __ldg(ap);
                        dst[i][1] = __ldg(ap + 1);
                        dst[i][2] = __ldg(ap + 2);
                    } else {
                        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(pr.alpha) + a));
                        dst[i][0] = v.x;
                        dst[i][1] = v.y;
                    }
                } else if (pr.blk_kind == B_I8) {
                    const uint8_t *ap = reinterpret_cast<const uint8_t *>(pr.alpha) + a * 3;
                    dst[i][0] = (uint32_t)__ldg(ap) | ((uint32_t)__ldg(ap + 1) << 8) | ((uint32_t)__ldg(ap + 2) << 16);
                } else {
                    dst[i][0] = __ldg(reinterpret_cast<const uint16_t *>(pr.alpha) + a);
                }
            }
        }
    };
    auto decode_mult = [&](uint32_t v) -> float {   // v: 16 bits (fp16 / three 3-bit exponents) or three int8 exponents
        if (pr.blk_kind == B_F16) return __half2float(__ushort_as_half((unsigned short)v));
        if (pr.blk_kind == B_U16) return (float)(1u << (v & 7u)) + (float)(1u << ((v >> 3) & 7u)) + (float)(1u << ((v >> 6) & 7u));
        float m = 0.f;
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            const int sft = (int)(int8_t)(v >> (8 * t));
            if (sft != -128) m += exp2f((float)sft);
        }
        return m;
    };
    auto store_block_mult = [&](const uint32_t(&src)[NVI][NVW], uint32_t buffer_off) {
#pragma unroll
        for (int i = 0; i < NVI; ++i) {
            int gi, c, b;
            item_coords(tid + 256 * i, gi, c, b);
            if (b < Q) {
                const uint32_t row0 = lut_s + buffer_off + (uint32_t)((b * 16 + gi) * LUT_ROW_BYTES + 128);
                if (blk_quads) {
                    uint32_t v[4];
                    if (pr.blk_kind == B_I8) {
                        v[0] = src[i][0];
                        v[1] = (src[i][0] >> 24) | (src[i][1] << 8);
                        v[2] = (src[i][1] >> 16) | (src[i][2] << 16);
                        v[3] = src[i][2] >> 8;
                    } else {
                        v[0] = src[i][0] & 0xFFFFu;
                        v[1] = src[i][0] >> 16;
                        v[2] = src[i][1] & 0xFFFFu;
                        v[3] = src[i][1] >> 16;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        sts_f32(row0 + (uint32_t)(k * LUT_ROW_BYTES + 4 * (c ^ (gi + k))), decode_mult(v[k]));
                } else {
                    sts_f32(row0 + (uint32_t)(4 * (c ^ gi)), decode_mult(src[i][0]));
                }
            }
        }
    };
    if constexpr (BLK) {
        if (kb_begin < kb_end) load_block_alpha(kb_begin, t_first, raw_next);
    }
    uint32_t mbuf = 0;  // byte offset of the multiplier buffer the current tile uses (two buffers, alternating)

    [[maybe_unused]] const long long t_wait0 = SAL_CYCLES();
    pdl_wait();  // activations, bias, y and the scratch buffer may be written by the previous kernel
    [[maybe_unused]] const long long t_wait1 = SAL_CYCLES();
    [[maybe_unused]] long long t_data = 0, t_build = 0;

    int st = 0;
    uint32_t phase = 0;
    // One K block: build its tables into half `PAR` of the table rows, then walk the column tiles.
    auto process_block = [&](int kb, auto par_tag) {
        constexpr int PAR = BLK ? 0 : decltype(par_tag)::value;
        if constexpr (BLK) consumer_barrier(NCW * 32);  // one set of tables: the previous K block must be finished by all
        [[maybe_unused]] const long long t_b0 = SAL_CYCLES();
        if (!SAL_ABLATED(P, 2)) build_block(kb, PAR, warp, std::integral_constant<int, NCW>{});
        consumer_barrier(NCW * 32);
        t_build += SAL_CYCLES() - t_b0;
        // The activations of the next K block are asked into L1 now, so that its table build does not start with
        // a trip to L2 (no registers held meanwhile; one 16-byte line piece per lane of one warp covers the block).
        if (SWIGLU == 0 && warp == 0 && kb + 1 < kb_end && !SAL_ABLATED(P, 128)) {
            const __half *nx0 = xrow0 + (size_t)(kb + 1) * KB_FEATS + 8 * lane;
            asm volatile("prefetch.global.L1 [%0];" ::"l"(nx0));
            if (ROWS == 2) asm volatile("prefetch.global.L1 [%0];" ::"l"(xrow1 + (size_t)(kb + 1) * KB_FEATS + 8 * lane));
        }
        // Rolled on purpose: the body is ~100 lookups long and exists once per table half;
        // unrolling it over the column tiles overflows the instruction cache.
        const int s_lo = kb == kb_begin ? t_first : 0, s_hi = kb == kb_last ? t_last + 1 : nsub;
#pragma unroll 1
        for (int sub = s_lo; sub < s_hi; ++sub) {
            __half a_cur[2][Q];
#pragma unroll
            for (int hp = 0; hp < 2; ++hp)
#pragma unroll
                for (int b = 0; b < Q; ++b) a_cur[hp][b] = a_next[hp][b];
            {
                const bool more_sub = (sub + 1 < s_hi);
                const int kb_n = more_sub ? kb : kb + 1;
                if constexpr (BLK) {
                    uint32_t raw_cur[NVI][NVW];
#pragma unroll
                    for (int i = 0; i < NVI; ++i)
#pragma unroll
                        for (int k = 0; k < NVW; ++k) raw_cur[i][k] = raw_next[i][k];
                    if (kb_n < kb_end && !SAL_ABLATED(P, 1)) load_block_alpha(kb_n, more_sub ? sub + 1 : 0, raw_next);
                    // Safe without a second barrier: whoever writes buffer `mbuf` again has passed the barrier of
                    // the tile in between, which every warp reaches only after its reads of this tile.
                    if (!SAL_ABLATED(P, 8)) store_block_mult(raw_cur, mbuf);
                    if (!SAL_ABLATED(P, 16)) consumer_barrier(NCW * 32);
                } else if (kb_n < kb_end && !SAL_ABLATED(P, 1)) {
                    load_alpha(kb_n, more_sub ? sub + 1 : 0, a_next);
                }
            }
            float a_sub[ROWS];
#pragma unroll
            for (int r = 0; r < ROWS; ++r) a_sub[r] = 0.f;
            constexpr int PPS = C::PPS;
            if constexpr (!BLK) {
#pragma unroll
                for (int b0 = 0; b0 < Q; b0 += PPS) {   // one ring slot: PPS planes of this unit
                    [[maybe_unused]] const long long t_d0 = SAL_CYCLES();
                    mbar_wait(full0 + 8 * st, phase, P.status);
                    t_data += SAL_CYCLES() - t_d0;
                    const uint32_t soff = (uint32_t)st * C::STAGE_BYTES;
                    if (!SAL_ABLATED(P, 4)) {
#pragma unroll
                        for (int hp = 0; hp < 2; ++hp) {
                            float part[ROWS][PPS], part2[ROWS][PPS];
#pragma unroll
                            for (int r = 0; r < ROWS; ++r)
#pragma unroll
                                for (int p = 0; p < PPS; ++p) part[r][p] = part2[r][p] = 0.f;
                            // all weight words of this half are requested before the first lookup
                            uint32_t wv[4][PPS];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t wr = wrow[hp][j] + soff;
#pragma unroll
                                for (int p = 0; p < PPS; ++p) {
                                    if (p == 0) wv[j][p] = lds_u32_imm<0>(wr);
                                    else if (p == 1) wv[j][p] = lds_u32_imm<1 * BOX_COLS * 4>(wr);
                                    else wv[j][p] = lds_u32_imm<2 * BOX_COLS * 4>(wr);
                                }
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
#pragma unroll
                                for (int p = 0; p < PPS; ++p) {
                                    const uint32_t w = wv[j][p];
                                    uint32_t e[4];
#pragma unroll
                                    for (int t = 0; t < 4; ++t) {
                                        const uint32_t off = prmt(w, cpack[hp][j], sel[t]);
                                        e[t] = ABS ? lds_u32_imm<(int)SMEM_DYNAMIC_BASE + PAR * 128>(off) : lds_u32_imm<0>(off + lut_s + PAR * 128);
                                    }
                                    if (ROWS == 1 && SAL_ABLATED(P, 64)) {   // timing only: integer adds (two entries per instruction)
                                        part[0][p] = __uint_as_float(__float_as_uint(part[0][p]) + e[0] + e[2]);
                                        part2[0][p] = __uint_as_float(__float_as_uint(part2[0][p]) + e[1] + e[3]);
                                    } else if (ROWS == 1) {
                                        part[0][p] += __uint_as_float(e[0]);
                                        part2[0][p] += __uint_as_float(e[1]);
                                        part[0][p] += __uint_as_float(e[2]);
                                        part2[0][p] += __uint_as_float(e[3]);
                                    } else {
                                        // four half2 entries are added in fp16 (they are bounded by 8 max|x| each), then
                                        // the word's sum is widened: fp32 carries everything beyond one weight word
                                        const __half2 s01 = __hadd2(*reinterpret_cast<const __half2 *>(&e[0]), *reinterpret_cast<const __half2 *>(&e[1]));
                                        const __half2 s23 = __hadd2(*reinterpret_cast<const __half2 *>(&e[2]), *reinterpret_cast<const __half2 *>(&e[3]));
                                        const float2 f = __half22float2(__hadd2(s01, s23));
                                        if (j & 1) {
                                            part2[0][p] += f.x;
                                            part2[ROWS - 1][p] += f.y;
                                        } else {
                                            part[0][p] += f.x;
                                            part[ROWS - 1][p] += f.y;
                                        }
                                    }
                                }
                            }
#pragma unroll
                            for (int p = 0; p < PPS; ++p) {
                                const float a = __half2float((hp ^ hw) ? a_cur[1][b0 + p] : a_cur[0][b0 + p]);  // slot hp holds group hp ^ hw
#pragma unroll
                                for (int r = 0; r < ROWS; ++r) a_sub[r] += a * (part[r][p] + part2[r][p]);
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty0 + 8 * st);
                    if (++st == stages) {
                        st = 0;
                        phase ^= 1u;
                    }
                }
            } else {
                // block mode walks the planes innermost (the multiplier addresses of a word are shared by its
                // planes): wait for all slots of the unit, hand them back at the end
                constexpr int SLOTS = C::SLOTS;
                uint32_t soffs[SLOTS];
                int st_b = st;
                uint32_t ph_b = phase;
#pragma unroll
                for (int i = 0; i < SLOTS; ++i) {
                    mbar_wait(full0 + 8 * st_b, ph_b, P.status);
                    soffs[i] = (uint32_t)st_b * C::STAGE_BYTES;
                    if (++st_b == stages) {
                        st_b = 0;
                        ph_b ^= 1u;
                    }
                }
                if (!SAL_ABLATED(P, 4))
#pragma unroll
                for (int hp = 0; hp < 2; ++hp) {
                    float part = 0.f, part2 = 0.f;
                    // all weight words of this half are requested before the first lookup, so that the (longer)
                    // chains table load -> multiplier load -> fma of one word overlap the next word's load
                    uint32_t wpre[4][Q];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int b = 0; b < Q; ++b) {
                            const uint32_t wr = wrow[hp][j] + soffs[b / PPS];
                            if (b % PPS == 0) wpre[j][b] = lds_u32_imm<0>(wr);
                            else if (b % PPS == 1) wpre[j][b] = lds_u32_imm<1 * BOX_COLS * 4>(wr);
                            else wpre[j][b] = lds_u32_imm<2 * BOX_COLS * 4>(wr);
                        }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // multiplier address: byte 0 <- 4 * (chunk ^ group), bytes 1.. <- row of (buffer, group)
                        const uint32_t rowsel = mrow + mbuf;
                        uint32_t ma[4];
                        ma[0] = prmt(mpack[hp][j], rowsel, 0x7650u) + (ABS ? 0u : lut_s);
                        ma[1] = prmt(mpack[hp][j], rowsel, 0x7651u) + (ABS ? 0u : lut_s);
                        ma[2] = prmt(mpack[hp][j], rowsel, 0x7652u) + (ABS ? 0u : lut_s);
                        ma[3] = prmt(mpack[hp][j], rowsel, 0x7653u) + (ABS ? 0u : lut_s);
#pragma unroll
                        for (int b = 0; b < Q; ++b) {
                            const uint32_t w = wpre[j][b];
                            uint32_t e[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const uint32_t off = prmt(w, cpack[hp][j], sel[t]);
                                e[t] = ABS ? lds_u32_imm<(int)SMEM_DYNAMIC_BASE + PAR * 128>(off) : lds_u32_imm<0>(off + lut_s + PAR * 128);
                            }
                            constexpr int MB = (ABS ? (int)SMEM_DYNAMIC_BASE : 0) + 128;
                            float m[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                if (b == 0) m[t] = lds_f32_imm<MB>(ma[t]);
                                else if (b == 1) m[t] = lds_f32_imm<MB + 1 * 16 * LUT_ROW_BYTES>(ma[t]);
                                else if (b == 2) m[t] = lds_f32_imm<MB + 2 * 16 * LUT_ROW_BYTES>(ma[t]);
                                else m[t] = lds_f32_imm<MB + 3 * 16 * LUT_ROW_BYTES>(ma[t]);
                            }
                            part = fmaf(m[0], __uint_as_float(e[0]), part);
                            part2 = fmaf(m[1], __uint_as_float(e[1]), part2);
                            part = fmaf(m[2], __uint_as_float(e[2]), part);
                            part2 = fmaf(m[3], __uint_as_float(e[3]), part2);
                        }
                    }
                    a_sub[0] += part + part2;  // the multipliers are already in
                }
                __syncwarp();
                if (lane == 0) {
                    int st_r = st;
#pragma unroll
                    for (int i = 0; i < SLOTS; ++i) {
                        mbar_arrive(empty0 + 8 * st_r);
                        if (++st_r == stages) st_r = 0;
                    }
                }
                st = st_b;
                phase = ph_b;
            }
            if constexpr (ROWS == 1) {
                // the tile's accumulator is picked with predicated adds, so that acc[] has static indices and stays in
                // registers (8 of them)
#pragma unroll
                for (int i = 0; i < MAX_SUB; ++i)
                    if (i == sub) acc[0][i] += a_sub[0];
            } else {
                // two rows: 16 accumulators would not fit next to the rest; acc[] is indexed dynamically and lives in
                // (L1-resident) local memory, two accesses per tile and row
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc[r][sub] += a_sub[r];
            }
            if constexpr (BLK) mbuf ^= (uint32_t)(Q * 16 * LUT_ROW_BYTES);
        }
    };
    for (int kb = kb_begin; kb < kb_end; kb += 2) {
        process_block(kb, std::integral_constant<int, 0>{});
        if (kb + 1 < kb_end) process_block(kb + 1, std::integral_constant<int, 1>{});
    }

    // ---------------------------------- epilogue ----------------------------------
#ifdef SAL_MEASURE
    if (lane == 0 && (warp == 0 || warp == NCW - 1) && blockIdx.x < 512 && blockIdx.y == 0) {
        unsigned long long *d = g_cta_timers + (size_t)(blockIdx.x * 2 + (warp ? 1 : 0)) * 8;
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        d[0] = (unsigned long long)(t_wait1 - t_wait0);
        d[1] = (unsigned long long)t_data;
        d[2] = (unsigned long long)t_build;
        d[3] = (unsigned long long)(SAL_CYCLES() - t_wait1);
        d[4] = (unsigned long long)(u_end - u_begin);
        d[5] = (unsigned long long)(kb_end - kb_begin);
        d[6] = smid;
        d[7] = (unsigned long long)pi;
    }
#endif
    if (ATOMIC) {
        // y is a 64-bit fixed-point accumulator: fire-and-forget integer reductions in L2, nothing to wait for, and
        // the sum does not depend on the order in which the CTAs arrive
        unsigned long long *yacc = reinterpret_cast<unsigned long long *>(pr.y);
#pragma unroll
        for (int sub = 0; sub < MAX_SUB; ++sub) {
            const int n = (sub_begin + sub) * CW + col;
            const bool touched = kb_begin != kb_last ? true : (sub >= t_first && sub <= t_last);
            if (sub < nsub && n < N && touched) {
                float v = acc[0][sub];
                if (pr.bias && u_begin <= sub && sub < u_end) v += __half2float(pr.bias[n]);  // the CTA holding unit (K block 0, sub)
                atomicAdd(yacc + n, to_fixed(v));
            }
        }
        return;
    }
    if (S == 1) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (r < rows_here) {
                __half *yrow = pr.y + (size_t)(row0 + r) * N;
#pragma unroll
                for (int sub = 0; sub < MAX_SUB; ++sub) {
                    const int n = (sub_begin + sub) * CW + col;
                    if (sub < nsub && n < N) {
                        float v = acc[r][sub];
                        if (pr.bias) v += __half2float(pr.bias[n]);
                        if (P.accumulate) v += __half2float(yrow[n]);
                        const __half hv = __float2half_rn(v);
                        yrow[n] = hv;
                    }
                }
            }
        }
        if (EXCH && P.ex.world > 1) {
            // second pass on purpose (each thread re-reads what it just wrote): keeps the peer pointers out of
            // the registers of the loop above
            for (int sub = 0; sub < nsub; ++sub) {
                const int n = (sub_begin + sub) * CW + col;
                if (n < N) push_to_peers(P.ex, pr.gather_off, N, n, pr.y[n]);
            }
            signal_peers(P.ex, tid, NCW * 32);
        }
        return;
    }
    // partial sums: [activation row][K split][N]; arrival counters: [row pair][column range]
    const int SP = max(pr.splits, pr.splits_last);  // stride of the partial sums: [row][SP][N]
    unsigned *counter = pr.counters + (size_t)blockIdx.y * pr.ranges + range;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        if (r < rows_here) {
            float *prow = pr.partials + ((size_t)(row0 + r) * SP + split) * N;
#pragma unroll
            for (int sub = 0; sub < MAX_SUB; ++sub) {
                const int n = (sub_begin + sub) * CW + col;
                if (sub < nsub && n < N) __stcg(prow + n, acc[r][sub]);
            }
        }
    }
    // Arrival: ONE acquire-release add per CTA after a CTA barrier.  The release is cumulative over the barrier (the
    // partial sums stored by the other threads happen before it), the acquire makes the partial sums of the CTAs that
    // arrived earlier visible to this CTA's threads behind the second barrier.  (A __threadfence() in each of the 256
    // threads on either side, as an earlier version had, made every thread wait for its own stores to settle.)
    consumer_barrier(NCW * 32);
    if (tid == 0) {
        unsigned old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
        s_last = (old == (unsigned)(S - 1));
    }
    consumer_barrier(NCW * 32);
    if (s_last) {
        // The last CTA of a column range to arrive sums the partials of all K splits in
        // ascending split order (fixed, hence deterministic).  Up to 4 column tiles x 16 splits
        // = 64 independent L2 loads are in flight per thread, so the whole reduction costs one
        // or two round trips instead of one per column tile.
        for (int r = 0; r < rows_here; ++r) {
            const float *pbase = pr.partials + (size_t)(row0 + r) * SP * N;
            __half *yrow = pr.y + (size_t)(row0 + r) * N;
            for (int sub0 = 0; sub0 < nsub; sub0 += 4) {
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                for (int s0 = 0; s0 < S; s0 += 16) {
                    float t[4][16];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int n = (sub_begin + sub0 + u) * CW + col;
                        const bool live = (sub0 + u < nsub) && (n < N);
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            t[u][i] = (live && s0 + i < S) ? __ldcg(pbase + (size_t)(s0 + i) * N + n) : 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[u] += t[u][i];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int n = (sub_begin + sub0 + u) * CW + col;
                    if (sub0 + u < nsub && n < N) {
                        float rsum = v[u];
                        if (pr.bias) rsum += __half2float(pr.bias[n]);
                        if (P.accumulate) rsum += __half2float(yrow[n]);
                        const __half hv = __float2half_rn(rsum);
                        yrow[n] = hv;
                    }
                }
            }
        }
        if (tid == 0) *counter = 0u;  // leave the scratch buffer ready for the next call
        if (EXCH && P.ex.world > 1) {
            for (int sub = 0; sub < nsub; ++sub) {
                const int n = (sub_begin + sub) * CW + col;
                if (n < N) push_to_peers(P.ex, pr.gather_off, N, n, pr.y[n]);
            }
            signal_peers(P.ex, tid, NCW * 32);
        }
    }
}

// Reports where dynamic shared memory starts for a kernel without static shared memory.
__global__ void smem_base_probe_kernel(uint32_t *out) {
    extern __shared__ __align__(128) unsigned char probe_smem[];
    if (threadIdx.x == 0) *out = smem_u32(probe_smem);
}

// ------------------------------------------------------------------------------------------
// generic kernel: any K % 32 == 0, any N, 1 <= M <= 64, all five alpha encodings
// ------------------------------------------------------------------------------------------
struct GenericParams {
    const uint32_t *bw;
    const void *alpha;
    const __half *q_bias;
    const __half *bias;
    const __half *x;
    __half *y;
    int M, K, N, q;
    int g;        // mode A: group size along K
    int ngroups;  // mode B: number of column groups
    int gs;       // mode B: columns per group
    int num_apot;
    int accumulate;
    int ksplit;          // K splits (grid.z); > 1 needs the scratch buffer below
    float *partials;     // [M][ksplit][N]
    unsigned *counters;  // [M][column blocks]
};

template <int KIND>
__device__ __forceinline__ float block_multiplier(const void *alpha, size_t idx, int num_apot) {
    if (KIND == B_F16) return __half2float(reinterpret_cast<const __half *>(alpha)[idx]);
    if (KIND == B_U16) {
        const unsigned a = reinterpret_cast<const uint16_t *>(alpha)[idx];
        return (float)(1u << (a & 7u)) + (float)(1u << ((a >> 3) & 7u)) + (float)(1u << ((a >> 6) & 7u));
    }
    const int8_t *a = reinterpret_cast<const int8_t *>(alpha) + idx * (size_t)num_apot;
    float m = 0.f;
    for (int t = 0; t < num_apot; ++t)
        if (a[t] != -128) m += exp2f((float)a[t]);
    return m;
}

template <int KIND>
__global__ void __launch_bounds__(128) lutgemv_generic_kernel(const GenericParams p) {
    __shared__ float lut[32][256];
    const int tid = threadIdx.x;
    const int n = blockIdx.x * 128 + tid;
    const int m = blockIdx.y;
    const __half *xrow = p.x + (size_t)m * p.K;
    const int kwords = p.K / 32;
    const int kblocks = (kwords + KB_WORDS - 1) / KB_WORDS;
    const int split = blockIdx.z;
    const int kb_begin = (int)(((long long)split * kblocks) / p.ksplit);
    const int kb_end = (int)(((long long)(split + 1) * kblocks) / p.ksplit);
    float acc = 0.f;
    // Block modes: the multipliers of one K block for this CTA's column groups are decoded once into
    // shared memory (32 chunks x q planes x up to 17 groups) instead of once per lookup.
    constexpr int MT_Q = 4, MT_G = 17;
    __shared__ float mult[(KIND >= B_F16) ? 32 : 1][(KIND >= B_F16) ? MT_Q : 1][(KIND >= B_F16) ? MT_G : 1];
    const int ng_first = (KIND >= B_F16) ? (blockIdx.x * 128) / p.gs : 0;
    const int ng_last = (KIND >= B_F16) ? (min(blockIdx.x * 128 + 127, p.N - 1)) / p.gs : 0;
    const int ng_cnt = ng_last - ng_first + 1;
    const bool use_mult_table = (KIND >= B_F16) && p.q <= MT_Q && ng_cnt <= MT_G;
    for (int kb = kb_begin; kb < kb_end; ++kb) {
        __syncthreads();
        if (use_mult_table) {
            const int total = 32 * p.q * ng_cnt;
            for (int e = tid; e < total; e += 128) {
                const int g = e % ng_cnt, b = (e / ng_cnt) % p.q, c = e / (ng_cnt * p.q);
                const int cg = kb * 32 + c;   // global chunk index
                float m = 0.f;
                if (cg * 8 < p.K) m = block_multiplier<KIND>(p.alpha, ((size_t)cg * p.q + b) * p.ngroups + ng_first + g, p.num_apot);
                mult[(KIND >= B_F16) ? c : 0][(KIND >= B_F16) ? b : 0][(KIND >= B_F16) ? g : 0] = m;
            }
        }
        {
            const int chunk = tid >> 2;
            const int k0 = kb * KB_FEATS + chunk * 8;
            float xf[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) xf[i] = (k0 + i < p.K) ? __half2float(xrow[k0 + i]) : 0.f;
            const int e0 = (tid & 3) * 64;
            for (int e = e0; e < e0 + 64; ++e) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) s += ((e >> i) & 1) ? xf[i] : -xf[i];
                lut[chunk][e] = s;
            }
        }
        __syncthreads();
        if (n < p.N) {
            for (int wi = 0; wi < KB_WORDS; ++wi) {
                const int kk = kb * KB_WORDS + wi;
                if (kk >= kwords) break;
                if (KIND == A_ROW_F16 || KIND == A_ROW_HALVING) {
                    const int grp = (kk * 32) / p.g;
                    if (KIND == A_ROW_HALVING) {
                        const float xs = lut[4 * wi][255] + lut[4 * wi + 1][255] + lut[4 * wi + 2][255] + lut[4 * wi + 3][255];
                        acc += __half2float(p.q_bias[(size_t)grp * p.N + n]) * xs;
                    }
                    float a_halving = (KIND == A_ROW_HALVING)
                                          ? __half2float(reinterpret_cast<const __half *>(p.alpha)[(size_t)grp * p.N + n])
                                          : 0.f;
                    for (int b = 0; b < p.q; ++b) {
                        const uint32_t w = p.bw[((size_t)kk * p.q + b) * p.N + n];
                        const float part = lut[4 * wi][w & 255u] + lut[4 * wi + 1][(w >> 8) & 255u] +
                                           lut[4 * wi + 2][(w >> 16) & 255u] + lut[4 * wi + 3][w >> 24];
                        float a;
                        if (KIND == A_ROW_HALVING) {
                            a_halving *= 0.5f;
                            a = a_halving;
                        } else {
                            a = __half2float(reinterpret_cast<const __half *>(p.alpha)[((size_t)grp * p.q + b) * p.N + n]);
                        }
                        acc += a * part;
                    }
                } else {
                    const int ng = n / p.gs;
                    for (int b = 0; b < p.q; ++b) {
                        const uint32_t w = p.bw[((size_t)kk * p.q + b) * p.N + n];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float mlt;
                            if (use_mult_table) {
                                mlt = mult[4 * wi + j][b][ng - ng_first];
                            } else {
                                const size_t aidx = ((size_t)(4 * kk + j) * p.q + b) * p.ngroups + ng;
                                mlt = block_multiplier<KIND>(p.alpha, aidx, p.num_apot);
                            }
                            acc += mlt * lut[4 * wi + j][(w >> (8 * j)) & 255u];
                        }
                    }
                }
            }
        }
    }
    if (p.ksplit == 1) {
        if (n < p.N) {
            float v = acc;
            if (p.bias) v += __half2float(p.bias[n]);
            __half *yp = p.y + (size_t)m * p.N + n;
            if (p.accumulate) v += __half2float(*yp);
            *yp = __float2half_rn(v);
        }
        return;
    }
    // deterministic split-K, same scheme as the tiled kernel: partial sums to the scratch buffer,
    // the last CTA of a (row, column block) to arrive adds them up in ascending split order
    __shared__ int s_last;
    float *prow = p.partials + ((size_t)m * p.ksplit) * p.N;
    if (n < p.N) __stcg(prow + (size_t)split * p.N + n, acc);
    __syncthreads();
    unsigned *counter = p.counters + (size_t)m * gridDim.x + blockIdx.x;
    if (tid == 0) {   // one acquire-release add per CTA behind the barrier (see the tiled kernel)
        unsigned old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
        s_last = (old == (unsigned)(p.ksplit - 1));
    }
    __syncthreads();
    if (s_last) {
        if (n < p.N) {
            float v = 0.f;
            for (int s0 = 0; s0 < p.ksplit; s0 += 8) {
                float t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = (s0 + i < p.ksplit) ? __ldcg(prow + (size_t)(s0 + i) * p.N + n) : 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) v += t[i];
            }
            if (p.bias) v += __half2float(p.bias[n]);
            __half *yp = p.y + (size_t)m * p.N + n;
            if (p.accumulate) v += __half2float(*yp);
            *yp = __float2half_rn(v);
        }
        if (tid == 0) *counter = 0u;
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
thread_local cudaError_t g_last_cuda_error = cudaSuccess;
inline bool cuda_ok(cudaError_t e) {
    if (e != cudaSuccess) g_last_cuda_error = e;
    return e == cudaSuccess;
}

struct DeviceInfo {
    int valid;
    int sms;
    int cc_major;
    int smem_optin;
    int smem_base;  // 0 = not probed yet, else the probed start of dynamic shared memory
};
DeviceInfo g_dev[64];

int device_info(DeviceInfo **out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SAL_E_DEVICE;
    DeviceInfo &d = g_dev[dev];
    if (!d.valid) {
        int sms = 0, maj = 0, optin = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return SAL_E_DEVICE;
        if (cudaDeviceGetAttribute(&maj, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return SAL_E_DEVICE;
        if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return SAL_E_DEVICE;
        d.sms = sms;
        d.cc_major = maj;
        d.smem_optin = optin;
        d.valid = 1;
    }
    *out = &d;
    return d.cc_major == 10 ? SAL_OK : SAL_E_DEVICE;
}

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }


int g_force_per = 0, g_force_splits = 0;  // measurement hooks: override the planner's choice

struct Plan {
    int ranges, splits, splits_last, nsub_per_range, nsub_total, kblocks;
    int ctas;
    double cost;
};

// Estimated time of one CTA, in units of (one 256-feature K block x one 256-column tile): `n` units of a
// range `w` tiles wide that `c` CTAs share.  Building the tables of a K block costs about 0.25 units (a run
// of n units touches about n / w + 1 blocks once it no longer starts on a block boundary); the split-K tail
// grows with the number of partial sums.  Calibrated on sweeps over the launch shapes of a LLaMA-2-7B block.
double g_cost_tb = 0.25, g_cost_r0 = 0.5, g_cost_r1 = 0.05, g_cost_rw = 0.025;  // model constants (sal_debug_set can override)
// The launch being planned adds into accumulators (SAL_OUT_FIXED_ATOMIC): no last CTA that sums splits x tiles partial
// sums, and a cheaper share per split (measured on a decoder's chain of launches: 8 % over the constants above).
thread_local bool g_plan_accumulating = false;
double g_cost_r1_acc = 0.02;   // (sal_debug_set "cost_r1_acc")
double cta_cost(double n, int w, int c) {
    double cost = n + g_cost_tb * (n / w + (c > 1 ? 1.0 : 0.0));
    if (c > 1) cost += g_cost_r0 + (g_plan_accumulating ? g_cost_r1_acc * c : g_cost_r1 * c + g_cost_rw * c * w);
    return cost;
}

// Fewest CTAs with which one problem stays within `bound` (estimated time per CTA), over all range widths.
// Returns false if no width does.
bool plan_problem(int K, int N, double bound, bool allow_split, int cw, Plan *out) {
    const int nsub_total = (N + cw - 1) / cw;
    const int kblocks = K / KB_FEATS;
    // smallest number of CTAs for a range of `units` units, `w` tiles wide; 0 = impossible
    const auto ctas_for = [&](int units, int w, double *cost) {
        const int cmax = allow_split ? (units < MAX_SPLIT ? units : MAX_SPLIT) : 1;
        for (int c = 1; c <= cmax; ++c) {
            if (g_force_splits > 0 && allow_split && c != (g_force_splits < cmax ? g_force_splits : cmax)) continue;
            const double t = cta_cost((double)((units + c - 1) / c), w, c);
            if (t <= bound) {
                *cost = t;
                return c;
            }
        }
        return 0;
    };
    bool found = false;
    Plan best{};
    for (int per = 1; per <= MAX_SUB && per <= nsub_total; ++per) {
        if (g_force_per > 0 && per != (g_force_per < nsub_total ? g_force_per : nsub_total)) continue;
        const int ranges = (nsub_total + per - 1) / per;
        const int w_last = nsub_total - (ranges - 1) * per;
        double cost_full = 0.0, cost_last = 0.0;
        const int c_last = ctas_for(w_last * kblocks, w_last, &cost_last);
        const int c_full = ranges > 1 ? ctas_for(per * kblocks, per, &cost_full) : 1;
        if (c_last == 0 || c_full == 0) continue;
        const int ctas = (ranges - 1) * c_full + c_last;
        const double cost = cost_full > cost_last ? cost_full : cost_last;
        if (!found || ctas < best.ctas || (ctas == best.ctas && cost < best.cost)) {
            best = Plan{ranges, ranges > 1 ? c_full : c_last, c_last, per, nsub_total, kblocks, ctas, cost};
            found = true;
        }
    }
    if (found) *out = best;
    return found;
}

// Plans all problems of a launch: the smallest bound on the per-CTA time for which the launch fits into
// `slots` resident CTAs (bisection; every CTA of every problem then has about the same amount of work).
// If not even single-CTA ranges fit, the launch runs in several waves.
bool plan_group_once(const sal_problem *problems, int count, int slots, bool allow_split, int cw, double bound, Plan *plans,
                     int *total) {
    *total = 0;
    for (int i = 0; i < count; ++i) {
        if (!plan_problem(problems[i].K, problems[i].N, bound, allow_split, cw, &plans[i])) return false;
        *total += plans[i].ctas;
    }
    return *total <= slots;
}

struct PlanCacheEntry {
    unsigned long long key;
    int count;
    Plan plans[SAL_MAX_GROUP];
};
PlanCacheEntry g_plan_cache[256];
std::mutex g_plan_mutex;

void plan_group(const sal_problem *problems, int count, int slots, bool allow_split, int cw, Plan *plans, bool accumulating) {
    g_plan_accumulating = accumulating;
    // the plan depends on the shapes only: remember it (planning costs a few hundred microseconds)
    unsigned long long key = 1469598103934665603ull;
    const auto mix = [&](long long v) { key = (key ^ (unsigned long long)v) * 1099511628211ull; };
    mix(count), mix(slots), mix(allow_split), mix(cw), mix(g_force_per), mix(g_force_splits), mix(accumulating);
    for (int i = 0; i < count; ++i) mix(problems[i].K), mix(problems[i].N);
    PlanCacheEntry &slot = g_plan_cache[key & 255];
    {
        std::lock_guard<std::mutex> lock(g_plan_mutex);
        if (slot.key == key && slot.count == count) {
            for (int i = 0; i < count; ++i) plans[i] = slot.plans[i];
            return;
        }
    }
    double units_total = 0, hi = 0;
    for (int i = 0; i < count; ++i) {
        const double u = (double)((problems[i].N + cw - 1) / cw) * (problems[i].K / KB_FEATS);
        units_total += u;
        const double worst = cta_cost((problems[i].K / KB_FEATS) * (double)MAX_SUB, 1, 1) + 4.0;
        if (worst > hi) hi = worst;
    }
    int total = 0;
    for (int waves = 1;; ++waves) {
        if (plan_group_once(problems, count, slots * waves, allow_split, cw, hi, plans, &total)) {
            double lo = units_total / (slots * waves);
            double up = hi;
            for (int it = 0; it < 40 && up - lo > 0.01; ++it) {
                const double mid = 0.5 * (lo + up);
                Plan trial[SAL_MAX_GROUP];
                if (plan_group_once(problems, count, slots * waves, allow_split, cw, mid, trial, &total)) up = mid;
                else lo = mid;
            }
            plan_group_once(problems, count, slots * waves, allow_split, cw, up, plans, &total);
            break;
        }
        if (waves >= 64) break;  // cannot happen for shapes that passed validation; plans hold the last attempt
    }
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    slot.key = key;
    slot.count = count;
    for (int i = 0; i < count; ++i) slot.plans[i] = plans[i];
}

int planes_per_slot(int q) { return q == 4 ? 2 : q; }
int stage_bytes_for(int q, int ncw) { return KB_WORDS * planes_per_slot(q) * ncw * 32 * 4; }

int g_stage_override = 0;  // measurement hooks (sal_debug_set)
int g_budget_pct = 0;  // 0 = as many CTAs as can be resident (CTAs per SM x 100 %)
int g_ablate = 0;
int g_full_sm = 0;  // measurement hook: let one CTA use a whole SM's shared memory (deeper ring, one CTA per SM)

// Ring depth: as many slots as fit in half of an SM's shared memory next to the 64 KB of
// tables, so that two CTAs (of this kernel or of the next one in the stream) are resident
// together.  Block mode holds all slots of a unit at once (two for q = 4).

int choose_stages(int q, int ncw, int smem_optin, int *smem_bytes) {
    const int sb = stage_bytes_for(q, ncw);
    const bool whole_sm = g_full_sm || ncw > 8;
    const int per_cta = whole_sm ? smem_optin : (smem_optin + 1024) / 2 - 1024;  // each resident CTA also reserves 1 KB
    int budget = per_cta - LUT_BYTES - 256 - ACT_BYTES;  // barriers, the reduction flag, one K block of staged activations
    int stages = budget / sb;
    if (stages > 8) stages = 8;
    if (g_stage_override > 0 && g_stage_override < stages) stages = g_stage_override;
    if (stages < q / planes_per_slot(q)) stages = q / planes_per_slot(q) <= budget / sb ? q / planes_per_slot(q) : 0;
    if (stages < 1) return 0;
    *smem_bytes = LUT_BYTES + stages * sb + 2 * stages * 8 + 16 + ACT_BYTES;   // tables, ring, its barriers, a flag, staged activations
    return stages;
}

int g_abs_override = -1;  // measurement hook: 0/1 forces the addressing variant

// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that the
// library does not link against libcuda.
typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                           const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                           CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                           CUtensorMapFloatOOBfill);
TensorMapEncodeTiledFn g_encode_tiled = nullptr;

int encode_weight_map(CUtensorMap *out, const void *bw, int K, int N, int q) {
    if (!g_encode_tiled) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (!cuda_ok(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres)) ||
            qres != cudaDriverEntryPointSuccess || fn == nullptr)
            return SAL_E_LAUNCH;
        g_encode_tiled = reinterpret_cast<TensorMapEncodeTiledFn>(fn);
    }
    // [K/32 words][q planes][N columns], innermost first; strides in bytes of all but the innermost dimension
    const cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)q, (cuuint64_t)(K / 32)};
    const cuuint64_t strides[2] = {(cuuint64_t)N * 4, (cuuint64_t)N * 4 * (cuuint64_t)q};  // N % 4 == 0 keeps them multiples of 16
    const cuuint32_t box[3] = {(cuuint32_t)BOX_COLS, (cuuint32_t)planes_per_slot(q), (cuuint32_t)KB_WORDS};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_encode_tiled(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(bw), dims, strides, box,
                                      estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? SAL_OK : SAL_E_LAUNCH;
}

template <int Q, int NCW, bool ABS, int ROWS, int SWIGLU, bool EXCH = false, bool ATOMIC = false, bool BLK = false>
cudaError_t launch_tiled_variant(const TileParams &P, int ctas, int row_groups, int smem, unsigned flags, cudaStream_t stream) {
    auto kern = lutgemv_tiled_kernel<Q, NCW, ABS, ROWS, SWIGLU, EXCH, ATOMIC, BLK>;
    static int configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas, (unsigned)row_groups);
    cfg.blockDim = dim3(TileCfg<Q, NCW>::THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (flags & SAL_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kern, P);
}

// swiglu: 0 plain activations, 1 silu(x)*x_mul with fp16 operands, 2 with fp32 operands
template <int Q, bool ABS>
cudaError_t launch_tiled_abs(const TileParams &P, int rows, int row_groups, int swiglu, bool atomic_out, int ctas, int smem,
                             unsigned flags, cudaStream_t stream) {
    if (P.p[0].blk_kind)  // block mode: one activation row per grid.y
        return launch_tiled_variant<Q, 8, ABS, 1, 0, false, false, true>(P, ctas, row_groups, smem, flags, stream);
    if (P.ex.world > 1)   // fused exchange: M = 1, plain activations (checked by the caller)
        return launch_tiled_variant<Q, 8, ABS, 1, 0, true>(P, ctas, 1, smem, flags, stream);
    if (rows == 2)
        return swiglu ? launch_tiled_variant<Q, 8, ABS, 2, 1>(P, ctas, row_groups, smem, flags, stream)
                      : launch_tiled_variant<Q, 8, ABS, 2, 0>(P, ctas, row_groups, smem, flags, stream);
    if (atomic_out) {
        if (swiglu == 2) return launch_tiled_variant<Q, 8, ABS, 1, 2, false, true>(P, ctas, 1, smem, flags, stream);
        if (swiglu == 1) return launch_tiled_variant<Q, 8, ABS, 1, 1, false, true>(P, ctas, 1, smem, flags, stream);
        return launch_tiled_variant<Q, 8, ABS, 1, 0, false, true>(P, ctas, 1, smem, flags, stream);
    }
    if (swiglu == 2) return launch_tiled_variant<Q, 8, ABS, 1, 2>(P, ctas, 1, smem, flags, stream);
    return swiglu ? launch_tiled_variant<Q, 8, ABS, 1, 1>(P, ctas, 1, smem, flags, stream)
                  : launch_tiled_variant<Q, 8, ABS, 1, 0>(P, ctas, 1, smem, flags, stream);
}

template <int Q>
cudaError_t launch_tiled(const TileParams &P, int ctas, int rows, int row_groups, int swiglu, bool atomic_out, int smem,
                         unsigned flags, bool abs_ok, cudaStream_t stream) {
    const bool use_abs = g_abs_override >= 0 ? (g_abs_override != 0) : abs_ok;
    return use_abs ? launch_tiled_abs<Q, true>(P, rows, row_groups, swiglu, atomic_out, ctas, smem, flags, stream)
                   : launch_tiled_abs<Q, false>(P, rows, row_groups, swiglu, atomic_out, ctas, smem, flags, stream);
}

bool tiled_eligible(const void *bw, const void *alpha, const void *bias, const void *x, const void *y, int M, int K,
                    int N, int q, int num_groups) {
    if (M < 1 || M > SAL_MAX_M || q < 1 || q > 4) return false;
    if (K % KB_FEATS != 0 || N % 8 != 0 || N < 8) return false;
    if (num_groups <= 0 || K % num_groups != 0) return false;
    const int g = K / num_groups;
    if (g % 128 != 0) return false;
    if (g != 128 && g % KB_FEATS != 0) return false;
    if (!aligned(bw, 16) || !aligned(alpha, 16) || !aligned(x, 16)) return false;
    (void)bias;
    (void)y;
    return true;
}

int validate_common(const void *bw, const void *alpha, const void *x, const void *y, int M, int K, int N, int q) {
    if (!bw || !alpha || !x || !y) return SAL_E_NULL;
    if (M < 1 || M > SAL_MAX_M || K <= 0 || N <= 0 || q < 1 || q > SAL_MAX_Q) return SAL_E_SHAPE;
    if (K % 32 != 0) return SAL_E_SHAPE;
    if (!aligned(bw, 4) || !aligned(x, 2) || !aligned(y, 2)) return SAL_E_ALIGN;
    return SAL_OK;
}

int run_generic(int kind, GenericParams p, void *workspace, size_t ws_bytes, cudaStream_t stream) {
    const int col_blocks = (p.N + 127) / 128;
    const int kblocks = (p.K / 32 + KB_WORDS - 1) / KB_WORDS;
    // K splits: aim at about four CTAs per SM; needs the scratch buffer (counters and partial sums)
    p.ksplit = 1;
    DeviceInfo *dev = nullptr;
    if (workspace && device_info(&dev) == SAL_OK) {
        int want = (4 * dev->sms + col_blocks * p.M - 1) / (col_blocks * p.M);
        if (want > kblocks) want = kblocks;
        if (want > MAX_SPLIT) want = MAX_SPLIT;
        const size_t need = WS_PARTIAL_OFFSET + (size_t)p.M * (size_t)p.N * MAX_SPLIT * sizeof(float);
        if (want > 1 && col_blocks * p.M <= WS_MAX_COUNTERS && ws_bytes >= need) {
            p.ksplit = want;
            p.counters = reinterpret_cast<unsigned *>(reinterpret_cast<char *>(workspace) + WS_HEADER_BYTES);
            p.partials = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + WS_PARTIAL_OFFSET);
        }
    }
    dim3 grid((unsigned)col_blocks, (unsigned)p.M, (unsigned)p.ksplit);
    switch (kind) {
        case A_ROW_F16: lutgemv_generic_kernel<A_ROW_F16><<<grid, 128, 0, stream>>>(p); break;
        case A_ROW_HALVING: lutgemv_generic_kernel<A_ROW_HALVING><<<grid, 128, 0, stream>>>(p); break;
        case B_F16: lutgemv_generic_kernel<B_F16><<<grid, 128, 0, stream>>>(p); break;
        case B_U16: lutgemv_generic_kernel<B_U16><<<grid, 128, 0, stream>>>(p); break;
        default: lutgemv_generic_kernel<B_I8><<<grid, 128, 0, stream>>>(p); break;
    }
    return cuda_ok(cudaGetLastError()) ? SAL_OK : SAL_E_LAUNCH;
}

// Block mode (alpha [K/8][q][N/gs]) of a problem handed to run_tiled_group.
struct BlockAlpha {
    int kind;  // B_F16, B_U16 or B_I8
    int ngroups, gs, num_apot;
};

bool block_tiled_eligible(const void *bw, const void *alpha, const void *x, int M, int K, int N, int q, int num_groups, int kind,
                          int num_apot) {
    if (M < 1 || M > SAL_MAX_M || q < 1 || q > 4) return false;
    if (K % KB_FEATS != 0 || N % 8 != 0 || N < 8) return false;
    if (num_groups <= 0 || N % num_groups != 0) return false;
    const int gs = N / num_groups;
    if (!(gs == 16 || gs == 32 || gs == 64 || gs == 128 || gs % BOX_COLS == 0)) return false;
    if (kind == B_I8 && num_apot != 3) return false;  // three exponents per multiplier, as the reference's LutLinear stores them
    // 16/32/64 columns per group: the kernel fetches four consecutive groups with one aligned 8- or 12-byte load
    if (gs < 128 && (num_groups % 4 != 0 || !aligned(alpha, 8))) return false;
    return aligned(bw, 16) && aligned(x, 16) && aligned(alpha, 2);
}

// A grouped launch of the tiled kernel, planned and marshalled but not yet bound to a scratch buffer: the
// kernel parameters (problems, work split, one encoded tensor map per problem), the launch geometry and, per
// problem, where its arrival counters and partial sums go inside whatever scratch buffer a launch is given.
struct BuiltLaunch {
    TileParams P;
    int q, ctas, rows, row_groups, swiglu, smem, writers, M;
    bool atomic_out;
    unsigned flags;
    int counter_off[SAL_MAX_GROUP];  // first arrival counter of the problem, -1 = the problem is not split along K
    size_t n_off[SAL_MAX_GROUP];     // columns of the problems before it (offset of its partial sums, in columns)
    size_t ws_need;                  // bytes of scratch a launch needs (0 = none)
};

// Plans and marshals one grouped launch (all problems share q, M and the activation form).  `allow_split`: a
// scratch buffer will be there at launch time, so K may be split.  `encode`: also encode the tensor maps (needs a
// CUDA context; false for the geometry-only query).
int build_tiled_group(const sal_problem *problems, int count, unsigned flags, bool allow_split, bool encode, const sal_exchange *ex,
                      const BlockAlpha *blk, BuiltLaunch *out) {
    DeviceInfo *dev = nullptr;
    if (encode) {
        int rc = device_info(&dev);
        if (rc != SAL_OK) return rc;
    }
    const int sms = dev ? dev->sms : 148;
    const int optin = dev ? dev->smem_optin : 232448;
    BuiltLaunch &L = *out;
    L = BuiltLaunch{};
    L.q = problems[0].q;
    L.flags = flags;
    // Activation rows: M = 1 runs the fp32-table kernel; 2 <= M <= 64 runs the half2-table variant,
    // one pair of rows per grid.y (all problems of a launch must agree on M).
    const int M = L.M = problems[0].M;
    L.rows = (M > 1 && !blk) ? 2 : 1;
    L.row_groups = (M + L.rows - 1) / L.rows;
    const int ncw = 8;   // consumer warps per CTA (a 16-warp, one-CTA-per-SM shape was measured and is not faster)
    // all problems of a launch must agree on the activation form
    L.atomic_out = (flags & SAL_OUT_FIXED_ATOMIC) != 0;
    L.swiglu = problems[0].x_mul == nullptr ? 0 : ((flags & SAL_SWIGLU_FIXED) ? 2 : 1);
    if ((L.atomic_out || L.swiglu == 2) && (M != 1 || ex)) return SAL_E_UNSUPPORTED;
    if (blk && (L.atomic_out || L.swiglu || ex || count != 1)) return SAL_E_UNSUPPORTED;
    const int cw = ncw * 32;
    const int ctas_per_sm = ncw > 8 ? 1 : 2;
    const int stages = choose_stages(L.q, ncw, optin, &L.smem);
    if (stages == 0) return SAL_E_UNSUPPORTED;

    TileParams &P = L.P;
    P.count = count;
    P.stages = stages;
    P.accumulate = (flags & SAL_ACCUMULATE) ? 1 : 0;
    P.ablate = g_ablate;
    if (ex) {
        if (ex->world < 2 || ex->world > SAL_MAX_PEERS || ex->rank < 0 || ex->rank >= ex->world || ex->slot < 0 || M != 1 ||
            !ex->gather_offsets)
            return SAL_E_SHAPE;
        P.ex.world = ex->world;
        P.ex.rank = ex->rank;
        P.ex.slot = ex->slot;
        for (int t = 0; t < ex->world; ++t) {
            if (!ex->peer_buffers[t] || !ex->peer_flags[t]) return SAL_E_NULL;
            P.ex.base[t] = reinterpret_cast<__half *>(ex->peer_buffers[t]);
            P.ex.flags[t] = reinterpret_cast<unsigned *>(ex->peer_flags[t]);
        }
    }

    // every CTA of the launch gets about the same amount of work, whatever problem it belongs to
    const int pct = g_budget_pct > 0 ? g_budget_pct : 100 * ctas_per_sm;
    int slots = (int)(sms * (pct / 100.0) / L.row_groups);   // row groups share the SMs
    if (slots < 4 * count) slots = 4 * count;
    Plan plans[SAL_MAX_GROUP];
    plan_group(problems, count, slots, allow_split || L.atomic_out, cw, plans, L.atomic_out);
    int cta = 0;
    int counter_off = 0;
    size_t n_off = 0;
    for (int i = 0; i < count; ++i) {
        const sal_problem &sp = problems[i];
        const Plan &pl = plans[i];
        TileProblem &tp = P.p[i];
        tp.bw = reinterpret_cast<const uint32_t *>(sp.bw);
        tp.alpha = reinterpret_cast<const __half *>(sp.alpha);
        tp.bias = reinterpret_cast<const __half *>(sp.bias);
        tp.x = reinterpret_cast<const __half *>(sp.x);
        tp.x_mul = reinterpret_cast<const __half *>(sp.x_mul);
        tp.y = reinterpret_cast<__half *>(sp.y);
        tp.K = sp.K;
        tp.N = sp.N;
        tp.M = sp.M;
        tp.g = blk ? KB_FEATS : sp.K / sp.num_groups;
        if (blk) {
            tp.blk_kind = blk->kind;
            tp.blk_gs = blk->gs;
            tp.blk_ngroups = blk->ngroups;
            tp.blk_apot = blk->num_apot;
        }
        tp.kblocks = pl.kblocks;
        tp.nsub_total = pl.nsub_total;
        tp.nsub_per_range = pl.nsub_per_range;
        tp.ranges = pl.ranges;
        tp.splits = pl.splits;
        tp.splits_last = pl.splits_last;
        tp.cta_begin = cta;
        tp.gather_off = ex ? (long long)ex->gather_offsets[i] : 0;
        L.writers += pl.ranges;  // one CTA per column range stores final outputs
        if (encode) {
            const int erc = encode_weight_map(&P.tmap[i], sp.bw, sp.K, sp.N, sp.q);
            if (erc != SAL_OK) return erc;
        }
        L.counter_off[i] = -1;
        L.n_off[i] = n_off;
        if ((pl.splits > 1 || pl.splits_last > 1) && !L.atomic_out) {
            if (counter_off + pl.ranges * L.row_groups > WS_MAX_COUNTERS) return SAL_E_WORKSPACE;
            L.ws_need = WS_PARTIAL_OFFSET + (n_off + (size_t)sp.N) * (size_t)M * MAX_SPLIT * sizeof(float);
            L.counter_off[i] = counter_off;
            counter_off += pl.ranges * L.row_groups;
        }
        n_off += (size_t)sp.N;
        cta += pl.ctas;
    }
    L.ctas = cta;
    return SAL_OK;
}

// Binds a built launch to a scratch buffer (and, for the fused exchange, to a counter slot) and enqueues it.
int launch_built(const BuiltLaunch &L, void *workspace, size_t ws_bytes, int slot, cudaStream_t stream) {
    DeviceInfo *dev = nullptr;
    int rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    if (L.ws_need > 0 && (workspace == nullptr || ws_bytes < L.ws_need)) return SAL_E_WORKSPACE;
    TileParams P = L.P;
    P.status = workspace ? reinterpret_cast<int *>(workspace) : nullptr;
    if (slot >= 0) P.ex.slot = slot;
    for (int i = 0; i < P.count; ++i) {
        if (L.counter_off[i] < 0) continue;
        P.p[i].counters = reinterpret_cast<unsigned *>(reinterpret_cast<char *>(workspace) + WS_HEADER_BYTES) + L.counter_off[i];
        P.p[i].partials = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + WS_PARTIAL_OFFSET) + L.n_off[i] * (size_t)L.M * MAX_SPLIT;
    }
    // The first call on a device that has a workspace probes where dynamic shared memory
    // starts (one tiny kernel on `stream`, read back synchronously); it must therefore not be
    // made under stream capture.  Until probed, the variant without baked-in addresses runs.
    if (dev->smem_base == 0 && workspace != nullptr) {
        uint32_t *probe = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(workspace) + 64);
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(stream, &cap);
        if (cap == cudaStreamCaptureStatusNone) {
            smem_base_probe_kernel<<<1, 32, 256, stream>>>(probe);
            uint32_t base = 0;
            if (cuda_ok(cudaMemcpyAsync(&base, probe, 4, cudaMemcpyDeviceToHost, stream)) &&
                cuda_ok(cudaStreamSynchronize(stream)))
                dev->smem_base = base ? (int)base : -1;
        }
    }
    const bool abs_ok = dev->smem_base == (int)SMEM_DYNAMIC_BASE;
    cudaError_t e;
    switch (L.q) {
        case 1: e = launch_tiled<1>(P, L.ctas, L.rows, L.row_groups, L.swiglu, L.atomic_out, L.smem, L.flags, abs_ok, stream); break;
        case 2: e = launch_tiled<2>(P, L.ctas, L.rows, L.row_groups, L.swiglu, L.atomic_out, L.smem, L.flags, abs_ok, stream); break;
        case 3: e = launch_tiled<3>(P, L.ctas, L.rows, L.row_groups, L.swiglu, L.atomic_out, L.smem, L.flags, abs_ok, stream); break;
        default: e = launch_tiled<4>(P, L.ctas, L.rows, L.row_groups, L.swiglu, L.atomic_out, L.smem, L.flags, abs_ok, stream); break;
    }
    return cuda_ok(e) ? SAL_OK : SAL_E_LAUNCH;
}

int run_tiled_group(const sal_problem *problems, int count, unsigned flags, void *workspace, size_t ws_bytes,
                    cudaStream_t stream, sal_plan_info *info_only, const sal_exchange *ex = nullptr, int *writers_out = nullptr,
                    const BlockAlpha *blk = nullptr) {
    BuiltLaunch L;
    const bool have_ws = workspace != nullptr && ws_bytes >= WS_PARTIAL_OFFSET;
    int rc = build_tiled_group(problems, count, flags, have_ws, info_only == nullptr, ex, blk, &L);
    if (rc != SAL_OK) return rc;
    if (writers_out) *writers_out = L.writers;
    if (info_only) {
        info_only->tiled = 1;
        info_only->ctas = L.ctas;
        info_only->ranges = L.P.p[0].ranges;
        info_only->splits = L.P.p[0].splits;
        info_only->stages = L.P.stages;
        info_only->smem_bytes = L.smem;
        return SAL_OK;
    }
    return launch_built(L, workspace, ws_bytes, -1, stream);
}

// Problems of one grouped call sorted into classes of equal plane count q (each class is one kernel launch),
// keeping the caller's order inside a class.  Returns the number of classes.
int split_by_q(const sal_problem *problems, int count, sal_problem (*classes)[SAL_MAX_GROUP], int *sizes, int (*index)[SAL_MAX_GROUP]) {
    int nclass = 0;
    for (int i = 0; i < count; ++i) {
        int c = 0;
        while (c < nclass && classes[c][0].q != problems[i].q) ++c;
        if (c == nclass) sizes[nclass++] = 0;
        if (index) index[c][sizes[c]] = i;
        classes[c][sizes[c]++] = problems[i];
    }
    return nclass;
}

int validate_grouped(const sal_problem *problems, int count, bool exchange) {
    if (!problems) return SAL_E_NULL;
    if (count < 1 || count > SAL_MAX_GROUP) return SAL_E_SHAPE;
    for (int i = 0; i < count; ++i) {
        const sal_problem &sp = problems[i];
        int rc = validate_common(sp.bw, sp.alpha, sp.x, sp.y, sp.M, sp.K, sp.N, sp.q);
        if (rc != SAL_OK) return rc;
        if (sp.num_groups <= 0 || sp.K % sp.num_groups != 0) return SAL_E_SHAPE;
        if (sp.M != problems[0].M) return SAL_E_UNSUPPORTED;
        if (exchange && (sp.M != 1 || sp.x_mul != nullptr)) return SAL_E_UNSUPPORTED;
        if (sp.x_mul && !aligned(sp.x_mul, 16)) return SAL_E_ALIGN;
        if ((sp.x_mul != nullptr) != (problems[0].x_mul != nullptr)) return SAL_E_UNSUPPORTED;
        if (!tiled_eligible(sp.bw, sp.alpha, sp.bias, sp.x, sp.y, sp.M, sp.K, sp.N, sp.q, sp.num_groups))
            return SAL_E_UNSUPPORTED;
    }
    return SAL_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------
extern "C" {

int sal_version(void) { return SAL_VERSION; }

const char *sal_status_string(int status) {
    switch (status) {
        case SAL_OK: return "ok";
        case SAL_E_NULL: return "null pointer";
        case SAL_E_SHAPE: return "unsupported or inconsistent shape";
        case SAL_E_ALIGN: return "misaligned pointer";
        case SAL_E_WORKSPACE: return "workspace missing or too small";
        case SAL_E_LAUNCH: return "CUDA launch failed";
        case SAL_E_UNSUPPORTED: return "not implemented for this configuration";
        case SAL_E_DEVICE: return "no compute-capability 10.x device is current";
        case SAL_E_TIMEOUT: return "a bounded device-side wait expired";
        default: return "unknown status";
    }
}

const char *sal_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda_error); }

int sal_device_ok(void) {
    DeviceInfo *d = nullptr;
    return device_info(&d);
}

size_t sal_workspace_bytes(int M, int N) {
    if (M < 1) M = 1;
    if (N < 1) N = 1;
    return WS_PARTIAL_OFFSET + (size_t)M * (size_t)N * MAX_SPLIT * sizeof(float);
}

int sal_workspace_status(void *workspace, void *stream) {
    if (!workspace) return SAL_E_NULL;
    int st = 0;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&st, workspace, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return SAL_E_LAUNCH;
    if (cudaStreamSynchronize(s) != cudaSuccess) return SAL_E_LAUNCH;
    if (st != 0) {
        if (cudaMemsetAsync(workspace, 0, sizeof(int), s) != cudaSuccess) return SAL_E_LAUNCH;
    }
    return st;
}

#ifdef SAL_MEASURE
int sal_debug_read(void *host, size_t bytes) {
    const size_t n = bytes < sizeof(g_cta_timers) ? bytes : sizeof(g_cta_timers);
    return cuda_ok(cudaMemcpyFromSymbol(host, g_cta_timers, n)) ? SAL_OK : SAL_E_LAUNCH;
}

int sal_debug_set(const char *key, int value) {
    if (!key) return SAL_E_NULL;
    const auto eq = [&](const char *k) {
        const char *a = key;
        while (*a && *a == *k) ++a, ++k;
        return *a == *k;
    };
    if (eq("stages")) g_stage_override = value;
    else if (eq("abs")) g_abs_override = value;
    else if (eq("ablate")) g_ablate = value;
    else if (eq("full_sm")) g_full_sm = value;
    else if (eq("force_per")) g_force_per = value;
    else if (eq("force_splits")) g_force_splits = value;
    else if (eq("budget_pct")) g_budget_pct = value > 0 ? value : 0;
    else if (eq("cost_tb")) g_cost_tb = value / 1000.0;
    else if (eq("cost_r0")) g_cost_r0 = value / 1000.0;
    else if (eq("cost_r1")) g_cost_r1 = value / 1000.0;
    else if (eq("cost_rw")) g_cost_rw = value / 1000.0;
    else if (eq("cost_r1_acc")) g_cost_r1_acc = value / 1000.0;
    else return SAL_E_UNSUPPORTED;
    {
        std::lock_guard<std::mutex> lock(g_plan_mutex);   // remembered plans were made under the old settings
        for (auto &e : g_plan_cache) e.key = 0, e.count = 0;
    }
    return SAL_OK;
}
#endif  // SAL_MEASURE

int sal_plan_shift_scale(int M, int K, int N, int q, int num_groups, sal_plan_info *out) {
    if (!out) return SAL_E_NULL;
    *out = sal_plan_info{};
    if (M < 1 || K <= 0 || N <= 0 || q < 1 || num_groups <= 0 || K % 32 || K % num_groups) return SAL_E_SHAPE;
    // alignment is assumed (fresh allocations are 256-byte aligned)
    if (!tiled_eligible(reinterpret_cast<void *>(16), reinterpret_cast<void *>(16), nullptr, reinterpret_cast<void *>(16),
                        nullptr, M, K, N, q, num_groups)) {
        out->tiled = 0;
        out->ctas = ((N + 127) / 128) * M;
        return SAL_OK;
    }
    sal_problem sp = {};
    sp.M = M;
    sp.K = K;
    sp.N = N;
    sp.q = q;
    sp.num_groups = num_groups;
    return run_tiled_group(&sp, 1, 0, reinterpret_cast<void *>(16), (size_t)1 << 40, nullptr, out);
}

int sal_lutgemv_shift_scale(const void *bw, const void *alpha, const void *bias, const void *x, void *y, int M, int K,
                            int N, int q, int num_groups, unsigned flags, void *workspace, size_t workspace_bytes,
                            void *stream) {
    int rc = validate_common(bw, alpha, x, y, M, K, N, q);
    if (rc != SAL_OK) return rc;
    if (num_groups <= 0 || K % num_groups != 0) return SAL_E_SHAPE;
    const int g = K / num_groups;
    if (g % 32 != 0) return SAL_E_SHAPE;
    if (!aligned(alpha, 2) || (bias && !aligned(bias, 2))) return SAL_E_ALIGN;
    DeviceInfo *dev = nullptr;
    rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!(flags & SAL_FORCE_GENERIC) && tiled_eligible(bw, alpha, bias, x, y, M, K, N, q, num_groups)) {
        sal_problem sp = {bw, alpha, bias, x, y, M, K, N, q, num_groups};
        rc = run_tiled_group(&sp, 1, flags, workspace, workspace_bytes, s, nullptr);
        // a scratch buffer that is too small for this shape (or more row pairs x column ranges than it has
        // arrival counters) is not an error for the reference-style call: the generic kernel takes it
        if (rc != SAL_E_WORKSPACE || (flags & (SAL_OUT_FIXED_ATOMIC | SAL_SWIGLU_FIXED))) return rc;
    }
    GenericParams p = {};
    p.bw = reinterpret_cast<const uint32_t *>(bw);
    p.alpha = alpha;
    p.bias = reinterpret_cast<const __half *>(bias);
    p.x = reinterpret_cast<const __half *>(x);
    p.y = reinterpret_cast<__half *>(y);
    p.M = M; p.K = K; p.N = N; p.q = q; p.g = g;
    p.accumulate = (flags & SAL_ACCUMULATE) ? 1 : 0;
    return run_generic(A_ROW_F16, p, workspace, workspace_bytes, s);
}

int sal_lutgemv_compute(const void *bw, const void *alpha, const void *q_bias, const void *bias, const void *x, void *y,
                        int M, int K, int N, int q, int num_groups, unsigned flags, void *workspace,
                        size_t workspace_bytes, void *stream) {
    int rc = validate_common(bw, alpha, x, y, M, K, N, q);
    if (rc != SAL_OK) return rc;
    if (!q_bias) return SAL_E_NULL;
    if (num_groups <= 0 || K % num_groups != 0) return SAL_E_SHAPE;
    const int g = K / num_groups;
    if (g % 32 != 0) return SAL_E_SHAPE;
    DeviceInfo *dev = nullptr;
    rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    GenericParams p = {};
    p.bw = reinterpret_cast<const uint32_t *>(bw);
    p.alpha = alpha;
    p.q_bias = reinterpret_cast<const __half *>(q_bias);
    p.bias = reinterpret_cast<const __half *>(bias);
    p.x = reinterpret_cast<const __half *>(x);
    p.y = reinterpret_cast<__half *>(y);
    p.M = M; p.K = K; p.N = N; p.q = q; p.g = g;
    p.accumulate = (flags & SAL_ACCUMULATE) ? 1 : 0;
    return run_generic(A_ROW_HALVING, p, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

static int block_entry(int kind, const void *bw, const void *alpha, const void *bias, const void *x, void *y, int M,
                       int K, int N, int q, int num_groups, int num_apot, unsigned flags, void *workspace,
                       size_t workspace_bytes, void *stream) {
    int rc = validate_common(bw, alpha, x, y, M, K, N, q);
    if (rc != SAL_OK) return rc;
    if (num_groups <= 0 || N % num_groups != 0) return SAL_E_SHAPE;
    if (kind == B_I8 && (num_apot < 1 || num_apot > 8)) return SAL_E_SHAPE;
    if (kind != B_I8 && !aligned(alpha, 2)) return SAL_E_ALIGN;
    DeviceInfo *dev = nullptr;
    rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    GenericParams p = {};
    p.bw = reinterpret_cast<const uint32_t *>(bw);
    p.alpha = alpha;
    p.bias = reinterpret_cast<const __half *>(bias);
    p.x = reinterpret_cast<const __half *>(x);
    p.y = reinterpret_cast<__half *>(y);
    p.M = M; p.K = K; p.N = N; p.q = q;
    p.ngroups = num_groups;
    p.gs = N / num_groups;
    p.num_apot = num_apot;
    p.accumulate = (flags & SAL_ACCUMULATE) ? 1 : 0;
    if (!(flags & SAL_FORCE_GENERIC) && block_tiled_eligible(bw, alpha, x, M, K, N, q, num_groups, kind, num_apot)) {
        sal_problem sp = {bw, alpha, bias, x, y, M, K, N, q, /*num_groups (unused in block mode)*/ 1};
        const BlockAlpha blk = {kind, num_groups, N / num_groups, num_apot};
        rc = run_tiled_group(&sp, 1, flags & (SAL_ACCUMULATE | SAL_PDL), workspace, workspace_bytes,
                             reinterpret_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr, &blk);
        // many rows x many column ranges can outgrow the arrival counters of the scratch buffer (one
        // counter per row and range in this mode): the generic kernel takes those
        if (rc != SAL_E_WORKSPACE) return rc;
    }
    return run_generic(kind, p, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int sal_lutgemm_block(const void *bw, const void *alpha, const void *bias, const void *x, void *y, int M, int K, int N,
                      int q, int num_groups, unsigned flags, void *workspace, size_t workspace_bytes, void *stream) {
    return block_entry(B_F16, bw, alpha, bias, x, y, M, K, N, q, num_groups, 0, flags, workspace, workspace_bytes, stream);
}

int sal_lutgemm_block_shift(const void *bw, const void *alpha_u16, const void *bias, const void *x, void *y, int M,
                            int K, int N, int q, int num_groups, unsigned flags, void *workspace,
                            size_t workspace_bytes, void *stream) {
    return block_entry(B_U16, bw, alpha_u16, bias, x, y, M, K, N, q, num_groups, 0, flags, workspace, workspace_bytes, stream);
}

int sal_lutgemm_block_shift_int8(const void *bw, const void *alpha_i8, const void *bias, const void *x, void *y, int M,
                                 int K, int N, int q, int num_groups, int num_apot, unsigned flags, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    return block_entry(B_I8, bw, alpha_i8, bias, x, y, M, K, N, q, num_groups, num_apot, flags, workspace, workspace_bytes, stream);
}

int sal_lutgemv_grouped(const sal_problem *problems, int count, unsigned flags, void *workspace,
                        size_t workspace_bytes, void *stream) {
    int rc = validate_grouped(problems, count, false);
    if (rc != SAL_OK) return rc;
    DeviceInfo *dev = nullptr;
    rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    // one kernel launch per plane count (a group of layers quantised to different widths: mixed precision)
    sal_problem classes[SAL_MAX_GROUP][SAL_MAX_GROUP];
    int sizes[SAL_MAX_GROUP];
    const int nclass = split_by_q(problems, count, classes, sizes, nullptr);
    for (int c = 0; c < nclass; ++c) {
        rc = run_tiled_group(classes[c], sizes[c], flags, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream), nullptr);
        if (rc != SAL_OK) return rc;
    }
    return SAL_OK;
}

int sal_lutgemv_grouped_exchange(const sal_problem *problems, int count, unsigned flags, void *workspace,
                                 size_t workspace_bytes, const sal_exchange *exchange, int *writers_out, void *stream) {
    if (!exchange) return SAL_E_NULL;
    int rc = validate_grouped(problems, count, true);
    if (rc != SAL_OK) return rc;
    if (!exchange->gather_offsets) return SAL_E_NULL;
    DeviceInfo *dev = nullptr;
    rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    sal_problem classes[SAL_MAX_GROUP][SAL_MAX_GROUP];
    int sizes[SAL_MAX_GROUP], index[SAL_MAX_GROUP][SAL_MAX_GROUP];
    const int nclass = split_by_q(problems, count, classes, sizes, index);
    int writers = 0;
    for (int c = 0; c < nclass; ++c) {
        long long offs[SAL_MAX_GROUP];
        for (int i = 0; i < sizes[c]; ++i) offs[i] = exchange->gather_offsets[index[c][i]];
        sal_exchange ex = *exchange;
        ex.gather_offsets = offs;
        int w = 0;
        rc = run_tiled_group(classes[c], sizes[c], flags, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream),
                             nullptr, &ex, &w);
        if (rc != SAL_OK) return rc;
        writers += w;
    }
    if (writers_out) *writers_out = writers;
    return SAL_OK;
}

// ---- prepared launches ----------------------------------------------------------------------
struct sal_prepared {
    int device;
    int nlaunch;
    int writers;
    size_t ws_need;
    BuiltLaunch launch[SAL_MAX_GROUP];
};

int sal_prepare_grouped(const sal_problem *problems, int count, unsigned flags, const sal_exchange *exchange,
                        sal_prepared **out) {
    if (!out) return SAL_E_NULL;
    *out = nullptr;
    int rc = validate_grouped(problems, count, exchange != nullptr);
    if (rc != SAL_OK) return rc;
    if (exchange && !exchange->gather_offsets) return SAL_E_NULL;
    DeviceInfo *dev = nullptr;
    rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    sal_prepared *h = new (std::nothrow) sal_prepared();
    if (!h) return SAL_E_LAUNCH;
    cudaGetDevice(&h->device);
    sal_problem classes[SAL_MAX_GROUP][SAL_MAX_GROUP];
    int sizes[SAL_MAX_GROUP], index[SAL_MAX_GROUP][SAL_MAX_GROUP];
    h->nlaunch = split_by_q(problems, count, classes, sizes, index);
    for (int c = 0; c < h->nlaunch; ++c) {
        long long offs[SAL_MAX_GROUP];
        sal_exchange ex;
        if (exchange) {
            for (int i = 0; i < sizes[c]; ++i) offs[i] = exchange->gather_offsets[index[c][i]];
            ex = *exchange;
            ex.gather_offsets = offs;
            if (ex.slot < 0) ex.slot = 0;
        }
        rc = build_tiled_group(classes[c], sizes[c], flags, true, true, exchange ? &ex : nullptr, nullptr, &h->launch[c]);
        if (rc != SAL_OK) {
            delete h;
            return rc;
        }
        h->writers += h->launch[c].writers;
        if (h->launch[c].ws_need > h->ws_need) h->ws_need = h->launch[c].ws_need;
    }
    *out = h;
    return SAL_OK;
}

size_t sal_prepared_workspace_bytes(const sal_prepared *prepared) { return prepared ? (prepared->ws_need ? prepared->ws_need : WS_PARTIAL_OFFSET) : 0; }

int sal_prepared_writers(const sal_prepared *prepared) { return prepared ? prepared->writers : 0; }

int sal_launch_prepared(const sal_prepared *prepared, void *workspace, size_t workspace_bytes, int slot, void *stream) {
    if (!prepared) return SAL_E_NULL;
    int dev = -1;
    if (!cuda_ok(cudaGetDevice(&dev)) || dev != prepared->device) return SAL_E_DEVICE;
    for (int c = 0; c < prepared->nlaunch; ++c) {
        const int rc = launch_built(prepared->launch[c], workspace, workspace_bytes, slot, reinterpret_cast<cudaStream_t>(stream));
        if (rc != SAL_OK) return rc;
    }
    return SAL_OK;
}

int sal_launch_prepared_sequence(const sal_prepared *const *prepared, int count, const int *slots, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    if (!prepared || count < 0) return SAL_E_NULL;
    for (int i = 0; i < count; ++i) {
        const int rc = sal_launch_prepared(prepared[i], workspace, workspace_bytes, slots ? slots[i] : -1, stream);
        if (rc != SAL_OK) return rc;
    }
    return SAL_OK;
}

void sal_destroy_prepared(sal_prepared *prepared) { delete prepared; }

int sal_exchange_wait(void *local_flags, int slot, unsigned expected, void *workspace, void *stream) {
    if (!local_flags) return SAL_E_NULL;
    if (slot < 0) return SAL_E_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_ok(cudaLaunchKernelEx(&cfg, exchange_wait_kernel, reinterpret_cast<unsigned *>(local_flags) + slot, expected,
                                      reinterpret_cast<int *>(workspace)))
               ? SAL_OK
               : SAL_E_LAUNCH;
}

// ---- entry point that allocates nothing ---------------------------------------------------
// Scratch for sal_lutgemv_shift_scale_static: lives in the library's own device image, so every
// GPU that loads the library carries these ~4 MB until the process exits.
#define SAL_STATIC_MAX_COLUMNS 16384
static __device__ __align__(256) unsigned char g_static_scratch[WS_PARTIAL_OFFSET +
                                                                (size_t)SAL_STATIC_MAX_COLUMNS * MAX_SPLIT * sizeof(float)];
static void *g_static_scratch_addr[64];  // device address of the array above, per device ordinal

int sal_lutgemv_shift_scale_static(const void *bw, const void *alpha, const void *bias, const void *x, void *y, int M,
                                   int K, int N, int q, int num_groups, unsigned flags, void *stream) {
    if (M < 1 || N < 1) return SAL_E_SHAPE;
    if ((long long)M * (long long)N > SAL_STATIC_MAX_COLUMNS) return SAL_E_WORKSPACE;  // beyond the built-in scratch
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev)) || dev < 0 || dev >= 64) return SAL_E_DEVICE;
    if (g_static_scratch_addr[dev] == nullptr) {
        // `g_static_scratch` names a host-side stand-in here; the device address has to be asked for,
        // with the device it is wanted for current (it is: cudaGetDevice above).
        void *addr = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&addr, g_static_scratch)) || addr == nullptr) return SAL_E_LAUNCH;
        g_static_scratch_addr[dev] = addr;
    }
    void *ws = g_static_scratch_addr[dev];
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left.  The arrival counters must start at zero (a call that
    // was cut short could have left them half way); the status word in the header is left alone, so that a
    // device-side SAL_E_TIMEOUT / SAL_E_UNSUPPORTED stays readable through sal_static_status.
    if (!cuda_ok(cudaMemsetAsync(static_cast<char *>(ws) + WS_HEADER_BYTES, 0, WS_COUNTER_BYTES, s))) return SAL_E_LAUNCH;
    return sal_lutgemv_shift_scale(bw, alpha, bias, x, y, M, K, N, q, num_groups, flags, ws, sizeof(g_static_scratch), s);
}

// Status word of the built-in scratch of the current device, read back (synchronously, on `stream`) and cleared.
int sal_static_status(void *stream) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev)) || dev < 0 || dev >= 64) return SAL_E_DEVICE;
    if (g_static_scratch_addr[dev] == nullptr) return SAL_OK;  // no call on this device yet: nothing recorded
    return sal_workspace_status(g_static_scratch_addr[dev], stream);
}

}  // extern "C"
