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
//   * one producer warp issues TMA bulk copies (cp.async.bulk + mbarrier
//     complete_tx) of [8 words][q planes][CW columns] weight tiles plus the
//     matching alpha rows into a multi-stage shared-memory ring.  The copies do
//     not depend on the activations, so under programmatic dependent launch
//     they are issued before griddepcontrol.wait and overlap the previous
//     kernel's tail;
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

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

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

struct TileProblem {
    const uint32_t *bw;
    const __half *alpha;
    const __half *bias;
    const __half *x;
    __half *y;
    float *partials;     // [splits][N]
    unsigned *counters;  // [ranges]
    int K, N;
    int g;               // group size along K, multiple of 128
    int kblocks;         // K / 256
    int nsub_total;      // ceil(N / CW)
    int nsub_per_range;
    int ranges, splits;
    int cta_begin;
    int pad_;
};

struct TileParams {
    TileProblem p[SAL_MAX_GROUP];
    int count;
    int stages;
    int accumulate;
    int *status;
};

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
__device__ __forceinline__ void tma_bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
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
    static constexpr int W_ROWS = KB_WORDS * Q;     // weight rows per stage
    static constexpr int W_BYTES = W_ROWS * CW * 4;
    static constexpr int A_ROWS = 2 * Q;            // alpha rows per stage (two groups at g = 128)
    static constexpr int A_BYTES = A_ROWS * CW * 2;
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    static constexpr int THREADS = (NCW + 1) * 32;
};

// Builds the 32 tables of one K block.  Lane = chunk; a warp handles groups of
// eight consecutive entries (entry >> 3 = hgrp).  Bank of every store = lane.
template <int NCW>
__device__ __forceinline__ void build_tables(const __half *__restrict__ xblk, unsigned char *lut_half, int warp,
                                             int lane) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(xblk) + lane);
    float xf[8];
    {
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            xf[2 * i] = f.x;
            xf[2 * i + 1] = f.y;
        }
    }
    float low[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        low[i] = ((i & 1) ? xf[0] : -xf[0]) + ((i & 2) ? xf[1] : -xf[1]) + ((i & 4) ? xf[2] : -xf[2]);
    float *dst = reinterpret_cast<float *>(lut_half) + lane;
#pragma unroll 1
    for (int hg = warp; hg < 32; hg += NCW) {
        const float hi = ((hg & 1) ? xf[3] : -xf[3]) + ((hg & 2) ? xf[4] : -xf[4]) + ((hg & 4) ? xf[5] : -xf[5]) +
                         ((hg & 8) ? xf[6] : -xf[6]) + ((hg & 16) ? xf[7] : -xf[7]);
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[(hg * 8 + i) * (LUT_ROW_BYTES / 4)] = hi + low[i];
    }
}

template <int Q, int NCW>
__global__ void __launch_bounds__(TileCfg<Q, NCW>::THREADS, 1)
    lutgemv_tiled_kernel(const __grid_constant__ TileParams P) {
    using C = TileCfg<Q, NCW>;
    constexpr int CW = C::CW;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ int s_last;

    unsigned char *lut = smem;
    unsigned char *stage_base = smem + LUT_BYTES;
    const int stages = P.stages;
    uint64_t *bars = reinterpret_cast<uint64_t *>(stage_base + (size_t)stages * C::STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + stages);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // which problem / column range / K split is this CTA
    int pi = 0;
#pragma unroll 1
    for (int i = 1; i < P.count; ++i)
        if ((int)blockIdx.x >= P.p[i].cta_begin) pi = i;
    const TileProblem &pr = P.p[pi];
    const int local = blockIdx.x - pr.cta_begin;
    const int range = local % pr.ranges;
    const int split = local / pr.ranges;
    const int N = pr.N;
    const int sub_begin = range * pr.nsub_per_range;
    const int nsub = min(pr.nsub_per_range, pr.nsub_total - sub_begin);
    const int kb_begin = (int)(((long long)split * pr.kblocks) / pr.splits);
    const int kb_end = (int)(((long long)(split + 1) * pr.kblocks) / pr.splits);
    const int gpk = (pr.g == 128) ? 2 : 1;  // groups per K block

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
        int it = 0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            const int grp0 = (kb * KB_FEATS) / pr.g;
            for (int sub = 0; sub < nsub; ++sub, ++it) {
                const int st = it % stages;
                const int use = it / stages;
                if (use > 0) mbar_wait(empty0 + 8 * st, (use - 1) & 1, P.status);
                const int n0 = (sub_begin + sub) * CW;
                const int valid = min(CW, N - n0);
                const uint32_t full = full0 + 8 * st;
                unsigned char *sdst = stage_base + (size_t)st * C::STAGE_BYTES;
                if (lane == 0) mbar_expect_tx(full, (uint32_t)(C::W_ROWS * valid * 4 + gpk * Q * valid * 2));
                __syncwarp();
                for (int row = lane; row < C::W_ROWS; row += 32) {
                    const uint32_t *src = pr.bw + ((size_t)kb * C::W_ROWS + row) * N + n0;
                    tma_bulk_g2s(smem_u32(sdst + (size_t)row * CW * 4), src, (uint32_t)valid * 4, full);
                }
                for (int row = lane; row < gpk * Q; row += 32) {
                    const __half *src = pr.alpha + ((size_t)grp0 * Q + row) * N + n0;
                    tma_bulk_g2s(smem_u32(sdst + C::W_BYTES + (size_t)row * CW * 2), src, (uint32_t)valid * 2, full);
                }
            }
        }
        return;
    }

    // -------------------------------- consumer warps --------------------------------
    const int col = warp * 32 + lane;
    const int hw = lane >> 4;
    const int rot = (lane >> 2) & 3;
    const int s4 = lane & 3;
    unsigned sel[4];
    unsigned coff[2][4][4];
    unsigned wrow[2][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) sel[t] = 4u | (unsigned)(((t + s4) & 3) << 4) | (6u << 8) | (7u << 12);
#pragma unroll
    for (int hp = 0; hp < 2; ++hp)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int wi = 4 * (hp ^ hw) + ((j + rot) & 3);
            wrow[hp][j] = (unsigned)(wi * Q * CW + col);
#pragma unroll
            for (int t = 0; t < 4; ++t) coff[hp][j][t] = (unsigned)(16 * wi + 4 * ((t + s4) & 3));
        }

    float acc[MAX_SUB];
#pragma unroll
    for (int i = 0; i < MAX_SUB; ++i) acc[i] = 0.f;

    pdl_wait();  // activations, bias, y and the scratch buffer may be written by the previous kernel

    int it = 0;
    for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int par = (kb - kb_begin) & 1;
        build_tables<NCW>(pr.x + (size_t)kb * KB_FEATS, lut + par * 128, warp, lane);
        consumer_barrier(NCW * 32);
        const unsigned char *lutp = lut + par * 128;
#pragma unroll
        for (int sub = 0; sub < MAX_SUB; ++sub) {
            if (sub < nsub) {
                const int st = it % stages;
                const int use = it / stages;
                ++it;
                mbar_wait(full0 + 8 * st, use & 1, P.status);
                const unsigned char *sdst = stage_base + (size_t)st * C::STAGE_BYTES;
                const uint32_t *wst = reinterpret_cast<const uint32_t *>(sdst);
                const __half *ast = reinterpret_cast<const __half *>(sdst + C::W_BYTES);
                float a_sub = 0.f;
#pragma unroll
                for (int hp = 0; hp < 2; ++hp) {
                    float part[Q];
#pragma unroll
                    for (int b = 0; b < Q; ++b) part[b] = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int b = 0; b < Q; ++b) {
                            const uint32_t w = wst[wrow[hp][j] + b * CW];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const unsigned addr = __byte_perm(w, coff[hp][j][t], sel[t]);
                                part[b] += *reinterpret_cast<const float *>(lutp + addr);
                            }
                        }
                    }
                    const int gl = (gpk == 2) ? (hp ^ hw) : 0;
#pragma unroll
                    for (int b = 0; b < Q; ++b) a_sub += __half2float(ast[(gl * Q + b) * CW + col]) * part[b];
                }
                acc[sub] += a_sub;
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * st);
            }
        }
    }

    // ---------------------------------- epilogue ----------------------------------
    if (pr.splits == 1) {
#pragma unroll
        for (int sub = 0; sub < MAX_SUB; ++sub) {
            const int n = (sub_begin + sub) * CW + col;
            if (sub < nsub && n < N) {
                float v = acc[sub];
                if (pr.bias) v += __half2float(pr.bias[n]);
                if (P.accumulate) v += __half2float(pr.y[n]);
                pr.y[n] = __float2half_rn(v);
            }
        }
        return;
    }
#pragma unroll
    for (int sub = 0; sub < MAX_SUB; ++sub) {
        const int n = (sub_begin + sub) * CW + col;
        if (sub < nsub && n < N) pr.partials[(size_t)split * N + n] = acc[sub];
    }
    __threadfence();
    consumer_barrier(NCW * 32);
    if (tid == 0) {
        const unsigned old = atomicAdd(&pr.counters[range], 1u);
        s_last = (old == (unsigned)(pr.splits - 1));
    }
    consumer_barrier(NCW * 32);
    if (s_last) {
        __threadfence();
        for (int sub = 0; sub < nsub; ++sub) {
            const int n = (sub_begin + sub) * CW + col;
            if (n < N) {
                float v = 0.f;
                for (int s = 0; s < pr.splits; ++s) v += __ldcg(&pr.partials[(size_t)s * N + n]);
                if (pr.bias) v += __half2float(pr.bias[n]);
                if (P.accumulate) v += __half2float(pr.y[n]);
                pr.y[n] = __float2half_rn(v);
            }
        }
        if (tid == 0) pr.counters[range] = 0u;  // leave the scratch buffer ready for the next call
    }
}

// ------------------------------------------------------------------------------------------
// generic kernel: any K % 32 == 0, any N, 1 <= M <= 64, all five alpha encodings
// ------------------------------------------------------------------------------------------
enum AlphaKind { A_ROW_F16 = 0, A_ROW_HALVING = 1, B_F16 = 2, B_U16 = 3, B_I8 = 4 };

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
    float acc = 0.f;
    for (int kb = 0; kb * KB_WORDS < kwords; ++kb) {
        __syncthreads();
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
                            const size_t aidx = ((size_t)(4 * kk + j) * p.q + b) * p.ngroups + ng;
                            acc += block_multiplier<KIND>(p.alpha, aidx, p.num_apot) * lut[4 * wi + j][(w >> (8 * j)) & 255u];
                        }
                    }
                }
            }
        }
    }
    if (n < p.N) {
        float v = acc;
        if (p.bias) v += __half2float(p.bias[n]);
        __half *yp = p.y + (size_t)m * p.N + n;
        if (p.accumulate) v += __half2float(*yp);
        *yp = __float2half_rn(v);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct DeviceInfo {
    int valid;
    int sms;
    int cc_major;
    int smem_optin;
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

constexpr int TILE_NCW = 8;
constexpr int TILE_CW = TILE_NCW * 32;

struct Plan {
    int ranges, splits, nsub_per_range, nsub_total, kblocks;
};

// Chooses column ranges x K splits for one problem given a CTA budget.
Plan plan_problem(int K, int N, int cta_budget, bool allow_split) {
    Plan best{};
    const int nsub_total = (N + TILE_CW - 1) / TILE_CW;
    const int kblocks = K / KB_FEATS;
    double best_cost = 1e30;
    for (int per = 1; per <= MAX_SUB && per <= nsub_total; ++per) {
        const int ranges = (nsub_total + per - 1) / per;
        int smax = allow_split ? (kblocks < MAX_SPLIT ? kblocks : MAX_SPLIT) : 1;
        for (int splits = 1; splits <= smax; ++splits) {
            const int ctas = ranges * splits;
            const int kb_per = (kblocks + splits - 1) / splits;
            const int waves = (ctas + cta_budget - 1) / cta_budget;
            // cost in "stage units": lookups + a table-build penalty per K block + a split penalty
            const double cost = waves * (kb_per * (per + 0.45)) + 0.02 * splits;
            if (cost < best_cost) {
                best_cost = cost;
                best = Plan{ranges, splits, per, nsub_total, kblocks};
            }
        }
    }
    return best;
}

template <int Q>
int tile_stage_bytes() {
    return TileCfg<Q, TILE_NCW>::STAGE_BYTES;
}
int stage_bytes_for(int q) {
    switch (q) {
        case 1: return tile_stage_bytes<1>();
        case 2: return tile_stage_bytes<2>();
        case 3: return tile_stage_bytes<3>();
        default: return tile_stage_bytes<4>();
    }
}

int g_stage_override = 0;  // test/benchmark hook (sal_debug_set_stages)

int choose_stages(int q, int smem_optin, int *smem_bytes) {
    const int sb = stage_bytes_for(q);
    int budget = smem_optin - LUT_BYTES - 256;
    int stages = budget / sb;
    if (stages > 8) stages = 8;
    if (g_stage_override > 0 && g_stage_override < stages) stages = g_stage_override;
    if (stages < 2) return 0;
    *smem_bytes = LUT_BYTES + stages * sb + 2 * stages * 8;
    return stages;
}

template <int Q>
cudaError_t launch_tiled(const TileParams &P, int ctas, int smem, unsigned flags, cudaStream_t stream) {
    auto kern = lutgemv_tiled_kernel<Q, TILE_NCW>;
    static int configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(TileCfg<Q, TILE_NCW>::THREADS);
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

bool tiled_eligible(const void *bw, const void *alpha, const void *bias, const void *x, const void *y, int M, int K,
                    int N, int q, int num_groups) {
    if (M != 1 || q < 1 || q > 4) return false;
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

int run_generic(int kind, const GenericParams &p, cudaStream_t stream) {
    dim3 grid((unsigned)((p.N + 127) / 128), (unsigned)p.M);
    switch (kind) {
        case A_ROW_F16: lutgemv_generic_kernel<A_ROW_F16><<<grid, 128, 0, stream>>>(p); break;
        case A_ROW_HALVING: lutgemv_generic_kernel<A_ROW_HALVING><<<grid, 128, 0, stream>>>(p); break;
        case B_F16: lutgemv_generic_kernel<B_F16><<<grid, 128, 0, stream>>>(p); break;
        case B_U16: lutgemv_generic_kernel<B_U16><<<grid, 128, 0, stream>>>(p); break;
        default: lutgemv_generic_kernel<B_I8><<<grid, 128, 0, stream>>>(p); break;
    }
    return cudaGetLastError() == cudaSuccess ? SAL_OK : SAL_E_LAUNCH;
}

int run_tiled_group(const sal_problem *problems, int count, unsigned flags, void *workspace, size_t ws_bytes,
                    cudaStream_t stream, sal_plan_info *info_only) {
    DeviceInfo *dev = nullptr;
    if (!info_only) {
        int rc = device_info(&dev);
        if (rc != SAL_OK) return rc;
    }
    const int sms = dev ? dev->sms : 148;
    const int optin = dev ? dev->smem_optin : 232448;
    const int q = problems[0].q;
    int smem = 0;
    const int stages = choose_stages(q, optin, &smem);
    if (stages == 0) return SAL_E_UNSUPPORTED;

    TileParams P = {};
    P.count = count;
    P.stages = stages;
    P.accumulate = (flags & SAL_ACCUMULATE) ? 1 : 0;
    P.status = workspace ? reinterpret_cast<int *>(workspace) : nullptr;

    // CTA budget per problem, proportional to its weight volume
    double units_total = 0;
    for (int i = 0; i < count; ++i)
        units_total += (double)((problems[i].N + TILE_CW - 1) / TILE_CW) * (problems[i].K / KB_FEATS);
    int cta = 0;
    int counter_off = 0;
    size_t n_off = 0;
    const bool have_ws = workspace != nullptr && ws_bytes >= WS_PARTIAL_OFFSET;
    for (int i = 0; i < count; ++i) {
        const sal_problem &sp = problems[i];
        const double units = (double)((sp.N + TILE_CW - 1) / TILE_CW) * (sp.K / KB_FEATS);
        int budget = (int)(sms * units / units_total + 0.5);
        if (budget < 1) budget = 1;
        Plan pl = plan_problem(sp.K, sp.N, budget, have_ws);
        TileProblem &tp = P.p[i];
        tp.bw = reinterpret_cast<const uint32_t *>(sp.bw);
        tp.alpha = reinterpret_cast<const __half *>(sp.alpha);
        tp.bias = reinterpret_cast<const __half *>(sp.bias);
        tp.x = reinterpret_cast<const __half *>(sp.x);
        tp.y = reinterpret_cast<__half *>(sp.y);
        tp.K = sp.K;
        tp.N = sp.N;
        tp.g = sp.K / sp.num_groups;
        tp.kblocks = pl.kblocks;
        tp.nsub_total = pl.nsub_total;
        tp.nsub_per_range = pl.nsub_per_range;
        tp.ranges = pl.ranges;
        tp.splits = pl.splits;
        tp.cta_begin = cta;
        if (pl.splits > 1) {
            if (counter_off + pl.ranges > WS_MAX_COUNTERS) return SAL_E_WORKSPACE;
            const size_t need = WS_PARTIAL_OFFSET + (n_off + (size_t)sp.N) * MAX_SPLIT * sizeof(float);
            if (!info_only && need > ws_bytes) return SAL_E_WORKSPACE;
            tp.counters = reinterpret_cast<unsigned *>(reinterpret_cast<char *>(workspace) + WS_HEADER_BYTES) + counter_off;
            tp.partials = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + WS_PARTIAL_OFFSET) + n_off * MAX_SPLIT;
            counter_off += pl.ranges;
        }
        n_off += (size_t)sp.N;
        cta += pl.ranges * pl.splits;
    }
    if (info_only) {
        info_only->tiled = 1;
        info_only->ctas = cta;
        info_only->ranges = P.p[0].ranges;
        info_only->splits = P.p[0].splits;
        info_only->stages = stages;
        info_only->smem_bytes = smem;
        return SAL_OK;
    }
    cudaError_t e;
    switch (q) {
        case 1: e = launch_tiled<1>(P, cta, smem, flags, stream); break;
        case 2: e = launch_tiled<2>(P, cta, smem, flags, stream); break;
        case 3: e = launch_tiled<3>(P, cta, smem, flags, stream); break;
        default: e = launch_tiled<4>(P, cta, smem, flags, stream); break;
    }
    return e == cudaSuccess ? SAL_OK : SAL_E_LAUNCH;
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

int sal_debug_set_stages(int stages) {
    g_stage_override = stages;
    return SAL_OK;
}

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
        return run_tiled_group(&sp, 1, flags, workspace, workspace_bytes, s, nullptr);
    }
    GenericParams p = {};
    p.bw = reinterpret_cast<const uint32_t *>(bw);
    p.alpha = alpha;
    p.bias = reinterpret_cast<const __half *>(bias);
    p.x = reinterpret_cast<const __half *>(x);
    p.y = reinterpret_cast<__half *>(y);
    p.M = M; p.K = K; p.N = N; p.q = q; p.g = g;
    p.accumulate = (flags & SAL_ACCUMULATE) ? 1 : 0;
    return run_generic(A_ROW_F16, p, s);
}

int sal_lutgemv_compute(const void *bw, const void *alpha, const void *q_bias, const void *bias, const void *x, void *y,
                        int M, int K, int N, int q, int num_groups, unsigned flags, void *workspace,
                        size_t workspace_bytes, void *stream) {
    (void)workspace;
    (void)workspace_bytes;
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
    return run_generic(A_ROW_HALVING, p, reinterpret_cast<cudaStream_t>(stream));
}

static int block_entry(int kind, const void *bw, const void *alpha, const void *bias, const void *x, void *y, int M,
                       int K, int N, int q, int num_groups, int num_apot, unsigned flags, void *stream) {
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
    return run_generic(kind, p, reinterpret_cast<cudaStream_t>(stream));
}

int sal_lutgemm_block(const void *bw, const void *alpha, const void *bias, const void *x, void *y, int M, int K, int N,
                      int q, int num_groups, unsigned flags, void *workspace, size_t workspace_bytes, void *stream) {
    (void)workspace;
    (void)workspace_bytes;
    return block_entry(B_F16, bw, alpha, bias, x, y, M, K, N, q, num_groups, 0, flags, stream);
}

int sal_lutgemm_block_shift(const void *bw, const void *alpha_u16, const void *bias, const void *x, void *y, int M,
                            int K, int N, int q, int num_groups, unsigned flags, void *workspace,
                            size_t workspace_bytes, void *stream) {
    (void)workspace;
    (void)workspace_bytes;
    return block_entry(B_U16, bw, alpha_u16, bias, x, y, M, K, N, q, num_groups, 0, flags, stream);
}

int sal_lutgemm_block_shift_int8(const void *bw, const void *alpha_i8, const void *bias, const void *x, void *y, int M,
                                 int K, int N, int q, int num_groups, int num_apot, unsigned flags, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    (void)workspace;
    (void)workspace_bytes;
    return block_entry(B_I8, bw, alpha_i8, bias, x, y, M, K, N, q, num_groups, num_apot, flags, stream);
}

int sal_lutgemv_grouped(const sal_problem *problems, int count, unsigned flags, void *workspace,
                        size_t workspace_bytes, void *stream) {
    if (!problems) return SAL_E_NULL;
    if (count < 1 || count > SAL_MAX_GROUP) return SAL_E_SHAPE;
    for (int i = 0; i < count; ++i) {
        const sal_problem &sp = problems[i];
        int rc = validate_common(sp.bw, sp.alpha, sp.x, sp.y, sp.M, sp.K, sp.N, sp.q);
        if (rc != SAL_OK) return rc;
        if (sp.num_groups <= 0 || sp.K % sp.num_groups != 0) return SAL_E_SHAPE;
        if (sp.q != problems[0].q) return SAL_E_UNSUPPORTED;
        if (!tiled_eligible(sp.bw, sp.alpha, sp.bias, sp.x, sp.y, sp.M, sp.K, sp.N, sp.q, sp.num_groups))
            return SAL_E_UNSUPPORTED;
    }
    DeviceInfo *dev = nullptr;
    int rc = device_info(&dev);
    if (rc != SAL_OK) return rc;
    return run_tiled_group(problems, count, flags, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream),
                           nullptr);
}

}  // extern "C"
