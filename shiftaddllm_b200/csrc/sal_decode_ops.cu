// Fused element-wise / attention steps of a batch-1 decode step (see include/sal_decode_ops.h).
// These are latency-bound helpers (a few KB each); the point is launch count, not bandwidth.
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sal_decode_ops.h"
#include "sal_lutgemm.h"

namespace {

// Fixed-point accumulators written by SAL_OUT_FIXED_ATOMIC products: signed 64-bit integers in units of 2**-32.
typedef long long acc_t;
__device__ __forceinline__ float acc_value(acc_t v) { return __ll2float_rn(v) * 2.3283064365386963e-10f; }


// Programmatic dependent launch: let the next kernel of the stream start (it may prefetch its
// constant operands), then wait until the previous kernel's results are visible.
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max over up to 1024 threads through one shared array of 32 floats.
__device__ __forceinline__ float block_reduce(float v, float *red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();  // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : (is_max ? -INFINITY : 0.f);
    r = is_max ? warp_max(r) : warp_sum(r);
    return r;
}

// Fast path of the norm kernels: at most 8 elements per thread, n a multiple of 8, 16-byte aligned operands.
__device__ __forceinline__ bool fast_rows_ok(int n, const void *a, const void *b, const void *c, const void *d, const void *e) {
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
                           reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(e);
    return (n % 8 == 0) && n <= 8 * (int)blockDim.x && (bits & 15) == 0;
}
// out[0..8) = t * inv * w (fp16), x_out[0..8) = t (fp16), one 16-byte store each
__device__ __forceinline__ void store_normed(const float (&t)[8], const uint4 &wv, float inv, __half *out, __half *x_out) {
    const __half *wh = reinterpret_cast<const __half *>(&wv);
    uint4 ov, xv;
    __half *oh = reinterpret_cast<__half *>(&ov), *xh = reinterpret_cast<__half *>(&xv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        oh[k] = __float2half_rn(t[k] * inv * __half2float(wh[k]));
        xh[k] = __float2half_rn(t[k]);
    }
    *reinterpret_cast<uint4 *>(out) = ov;
    if (x_out) *reinterpret_cast<uint4 *>(x_out) = xv;
}

__global__ void __launch_bounds__(1024) residual_rmsnorm_kernel(const __half *x, const __half *delta, const __half *w,
                                                                __half *out, __half *x_out, int n, float eps) {
    __shared__ float red[32];
    extern __shared__ float tbuf[];  // n floats
    pdl_prologue();
    {   // one CTA per row (grid.x rows of n elements each; the weight is shared)
        const size_t row = (size_t)blockIdx.x * n;
        x += row;
        out += row;
        if (delta) delta += row;
        if (x_out) x_out += row;
    }
    if (fast_rows_ok(n, x, delta, w, out, x_out)) {
        // n <= 8 x threads, everything 16-byte aligned: a thread keeps its 8 elements in registers, every
        // operand is fetched with one 16-byte load and all loads are in flight together
        const int i = threadIdx.x * 8;
        const bool mine = i < n;
        float t[8];
        uint4 wv = make_uint4(0u, 0u, 0u, 0u);
        if (mine) {
            const uint4 xv = *reinterpret_cast<const uint4 *>(x + i);
            wv = *reinterpret_cast<const uint4 *>(w + i);
            uint4 dv = make_uint4(0u, 0u, 0u, 0u);
            if (delta) dv = *reinterpret_cast<const uint4 *>(delta + i);
            const __half *xh = reinterpret_cast<const __half *>(&xv), *dh = reinterpret_cast<const __half *>(&dv);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                t[k] = __half2float(xh[k]);
                if (delta) t[k] = __half2float(__float2half_rn(t[k] + __half2float(dh[k])));
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = 0.f;
        }
        float ssq = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ssq += t[k] * t[k];
        ssq = block_reduce(ssq, red, false);
        const float inv_f = rsqrtf(ssq / (float)n + eps);
        if (mine) store_normed(t, wv, inv_f, out + i, x_out ? x_out + i : nullptr);
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float t = __half2float(x[i]);
        if (delta) t = __half2float(__float2half_rn(t + __half2float(delta[i])));  // the stream is kept in fp16
        tbuf[i] = t;
        ss += t * t;
    }
    ss = block_reduce(ss, red, false);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float t = tbuf[i];
        if (x_out) x_out[i] = __float2half_rn(t);
        out[i] = __float2half_rn(t * inv * __half2float(w[i]));
    }
}

// Accumulator variant: delta is a fixed-point accumulator vector written by SAL_OUT_FIXED_ATOMIC products; it is
// rounded to fp16 (what the fp16-output path would have stored), consumed, and zeroed for its next use, together
// with up to two more accumulator vectors whose consumers (many CTAs of a GEMV) could not zero them themselves.
__global__ void __launch_bounds__(1024) residual_rmsnorm_acc_kernel(const __half *x, acc_t *delta, const __half *w, __half *out,
                                                                    __half *x_out, int n, float eps, acc_t *zero_a, int zero_a_n,
                                                                    acc_t *zero_b, int zero_b_n) {
    __shared__ float red[32];
    extern __shared__ float tbuf[];  // n floats
    pdl_prologue();
    if (blockIdx.x > 0) {
        // CTAs 1.. only clear the extra accumulators (hundreds of KB for an FFN-wide pair): nothing here depends
        // on the norm, so it runs beside it instead of in front of it
        const int stride = (gridDim.x - 1) * blockDim.x, first = (blockIdx.x - 1) * blockDim.x + threadIdx.x;
        for (int i = first; i < zero_a_n; i += stride) zero_a[i] = 0;
        for (int i = first; i < zero_b_n; i += stride) zero_b[i] = 0;
        return;
    }
    if (fast_rows_ok(n, x, delta, w, out, x_out)) {
        const int i = threadIdx.x * 8;
        const bool mine = i < n;
        float t[8];
        uint4 wv = make_uint4(0u, 0u, 0u, 0u);
        if (mine) {
            const uint4 xv = *reinterpret_cast<const uint4 *>(x + i);
            wv = *reinterpret_cast<const uint4 *>(w + i);
            float df[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (delta) {
                longlong2 d[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) d[k] = *reinterpret_cast<const longlong2 *>(delta + i + 2 * k);   // 16-byte loads, all in flight
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    *reinterpret_cast<longlong2 *>(delta + i + 2 * k) = make_longlong2(0, 0);
                    df[2 * k] = acc_value(d[k].x);
                    df[2 * k + 1] = acc_value(d[k].y);
                }
            }
            const __half *xh = reinterpret_cast<const __half *>(&xv);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                t[k] = __half2float(xh[k]);
                if (delta) t[k] = __half2float(__float2half_rn(t[k] + __half2float(__float2half_rn(df[k]))));
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = 0.f;
        }
        float ssq = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ssq += t[k] * t[k];
        ssq = block_reduce(ssq, red, false);
        const float inv_f = rsqrtf(ssq / (float)n + eps);
        if (mine) store_normed(t, wv, inv_f, out + i, x_out ? x_out + i : nullptr);
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float t = __half2float(x[i]);
        if (delta) {
            t = __half2float(__float2half_rn(t + __half2float(__float2half_rn(acc_value(delta[i])))));
            delta[i] = 0;
        }
        tbuf[i] = t;
        ss += t * t;
    }
    ss = block_reduce(ss, red, false);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float t = tbuf[i];
        if (x_out) x_out[i] = __float2half_rn(t);
        out[i] = __float2half_rn(t * inv * __half2float(w[i]));
    }
}

// Accumulator variant of the rotary step: q, k, v are fixed-point accumulators (rounded to fp16 on read, then
// zeroed); the rotated query goes to q_out (fp16), rotated k and v to the caches.
__global__ void rope_kv_write_acc_kernel(acc_t *q, acc_t *k, acc_t *v, __half *q_out, const float *cos_t, const float *sin_t,
                                         const int64_t *pos_p, __half *k_cache, __half *v_cache, int heads, int kv_heads,
                                         int hd, int max_len) {
    pdl_prologue();
    const int64_t pos = *pos_p;
    if (pos < 0 || pos >= max_len) return;
    const int half = hd / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int nq = heads * half, nk = kv_heads * half, nv = kv_heads * hd;
    if (idx < nq + nk) {
        const bool is_q = idx < nq;
        const int j = is_q ? idx : idx - nq;
        const int h = j / half, i = j % half;
        const float c = cos_t[pos * half + i], s = sin_t[pos * half + i];
        acc_t *src = is_q ? q : k;
        const float a = __half2float(__float2half_rn(acc_value(src[h * hd + i])));
        const float b = __half2float(__float2half_rn(acc_value(src[h * hd + half + i])));
        src[h * hd + i] = 0;
        src[h * hd + half + i] = 0;
        const __half ra = __float2half_rn(a * c - b * s), rb = __float2half_rn(b * c + a * s);
        __half *dst = is_q ? q_out : k_cache + ((size_t)pos * kv_heads) * hd;
        dst[h * hd + i] = ra;
        dst[h * hd + half + i] = rb;
    } else if (idx < nq + nk + nv) {
        const int j = idx - nq - nk;
        v_cache[(size_t)pos * kv_heads * hd + j] = __float2half_rn(acc_value(v[j]));
        v[j] = 0;
    }
}

// one thread per (head, pair index); q heads first, then k heads, then v copy
__global__ void rope_kv_write_kernel(__half *q, const __half *k, const __half *v, const float *cos_t, const float *sin_t,
                                     const int64_t *pos_p, __half *k_cache, __half *v_cache, int heads, int kv_heads,
                                     int hd, int max_len) {
    pdl_prologue();
    const int64_t pos = *pos_p;
    if (pos < 0 || pos >= max_len) return;
    const int half = hd / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int nq = heads * half, nk = kv_heads * half, nv = kv_heads * hd;
    if (idx < nq + nk) {
        const bool is_q = idx < nq;
        const int j = is_q ? idx : idx - nq;
        const int h = j / half, i = j % half;
        const float c = cos_t[pos * half + i], s = sin_t[pos * half + i];
        const __half *src = is_q ? q : k;
        const float a = __half2float(src[h * hd + i]), b = __half2float(src[h * hd + half + i]);
        const __half ra = __float2half_rn(a * c - b * s), rb = __float2half_rn(b * c + a * s);
        __half *dst = is_q ? q : k_cache + ((size_t)pos * kv_heads) * hd;
        dst[h * hd + i] = ra;
        dst[h * hd + half + i] = rb;
    } else if (idx < nq + nk + nv) {
        const int j = idx - nq - nk;
        v_cache[(size_t)pos * kv_heads * hd + j] = v[j];
    }
}

// one CTA per query head; scores for the T = pos+1 cached positions live in shared memory
__global__ void __launch_bounds__(1024) attention_decode_kernel(const __half *q, const __half *k_cache, const __half *v_cache,
                                                               const int64_t *pos_p, __half *out, int heads, int kv_heads,
                                                               int hd, int max_len, float scale) {
    extern __shared__ float smem_f[];  // hd floats (query) + max_len floats (scores) + 32*hd floats (partial outputs)
    __shared__ float red[32];
    pdl_prologue();
    float *qf = smem_f;
    float *sc = smem_f + hd;
    float *pbuf = sc + max_len;   // [warps][hd] partial outputs
    const int head = blockIdx.x;
    const int kvh = head / (heads / kv_heads);
    int64_t pos = *pos_p;
    if (pos >= max_len) pos = max_len - 1;
    const int T = (int)pos + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    for (int i = tid; i < hd; i += blockDim.x) qf[i] = __half2float(q[head * hd + i]) * scale;
    __syncthreads();
    // scores: one warp per cached position, lanes over the head dimension; four positions are
    // fetched before any of them is reduced, so that four row reads per warp are in flight
    float lmax = -INFINITY;
    for (int t0 = warp; t0 < T; t0 += 4 * nw) {
        float d[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int t = t0 + u * nw;
            d[u] = 0.f;
            if (t < T) {
                const __half *kr = k_cache + ((size_t)t * kv_heads + kvh) * hd;
                for (int i = lane * 2; i < hd; i += 64) {
                    const float2 kk = __half22float2(*reinterpret_cast<const __half2 *>(kr + i));
                    d[u] += qf[i] * kk.x + qf[i + 1] * kk.y;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int t = t0 + u * nw;
            const float r = warp_sum(d[u]);
            if (t < T) {
                if (lane == 0) sc[t] = r;
                lmax = fmaxf(lmax, r);
            }
        }
    }
    const float m = block_reduce(lmax, red, true);  // also publishes sc[] (barriers inside)
    float lsum = 0.f;
    for (int t = tid; t < T; t += blockDim.x) {
        const float p = __expf(sc[t] - m);
        sc[t] = p;
        lsum += p;
    }
    const float denom = block_reduce(lsum, red, false);
    __syncthreads();
    // output: every warp takes every nw-th position (one coalesced row read each, many in flight),
    // lanes over the head dimension; the per-warp partial outputs are then added up in shared memory
    float2 o[4];   // hd <= 256: up to four half2 per lane
#pragma unroll
    for (int u = 0; u < 4; ++u) o[u] = make_float2(0.f, 0.f);
    for (int t0 = warp; t0 < T; t0 += 4 * nw) {
        float2 vv[4][4];
        float p[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {          // issue the row reads of four positions first
            const int t = t0 + k * nw;
            p[k] = (t < T) ? sc[t] : 0.f;
            const __half *vr = v_cache + ((size_t)(t < T ? t : 0) * kv_heads + kvh) * hd;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = lane * 2 + u * 64;
                vv[k][u] = (i < hd) ? __half22float2(*reinterpret_cast<const __half2 *>(vr + i)) : make_float2(0.f, 0.f);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                o[u].x += p[k] * vv[k][u].x;
                o[u].y += p[k] * vv[k][u].y;
            }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = lane * 2 + u * 64;
        if (i < hd) {
            pbuf[warp * hd + i] = o[u].x;
            pbuf[warp * hd + i + 1] = o[u].y;
        }
    }
    __syncthreads();
    for (int i = tid; i < hd; i += blockDim.x) {
        float r = 0.f;
        for (int w = 0; w < nw; ++w) r += pbuf[w * hd + i];
        out[head * hd + i] = __float2half_rn(r / denom);
    }
}

// Greedy end of a step: fp32 copy of the fp16 logits, argmax (smallest index among equal maxima), position + 1.
__global__ void __launch_bounds__(1024) greedy_token_kernel(const __half *logits, float *logits32, int vocab, int64_t *token,
                                                            int64_t *pos) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_prologue();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {   // ascending indices per thread: '>' keeps the first
        const uint4 raw = *reinterpret_cast<const uint4 *>(logits + i);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
        float f[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 v = __half22float2(h[k]);
            f[2 * k] = v.x;
            f[2 * k + 1] = v.y;
        }
        if (logits32) {
            *reinterpret_cast<float4 *>(logits32 + i) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4 *>(logits32 + i + 4) = make_float4(f[4], f[5], f[6], f[7]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (f[k] > best) best = f[k], best_i = i + k;
    }
    // larger value wins, equal values: smaller index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) s_val[warp] = best, s_idx[warp] = best_i;
    __syncthreads();
    if (warp == 0) {
        best = lane < nw ? s_val[lane] : -INFINITY;
        best_i = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
        }
        if (lane == 0) {
            *token = best_i == 0x7fffffff ? 0 : best_i;   // all NaN or -inf: index 0
            *pos += 1;
        }
    }
}

__global__ void silu_mul_kernel(const __half *gate, const __half *up, __half *out, int n) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float g = __half2float(gate[i]);
        out[i] = __float2half_rn(__half2float(__float2half_rn(g / (1.f + __expf(-g)))) * __half2float(up[i]));
    }
}

// All helpers are launched with the programmatic-stream-serialization attribute (see pdl_prologue).
template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, void *stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) == cudaSuccess ? SAL_OK : SAL_E_LAUNCH;
}


// Single-query attention split over the cached positions ("flash decoding"): CTA (kv head, slice) handles
// the slice's positions for the G query heads that share the kv head, so a K or V row is read once per
// group.  A row of hd halves is read by hd/8 lanes with 16-byte loads (a warp covers 32/(hd/8) positions
// per load instruction, four instructions in flight).  Every CTA leaves (max, sum, unnormalised output)
// per query head in the scratch buffer; the last CTA of a kv head to arrive merges the slices.
constexpr int ATTN_MAX_SPLIT = 32;
constexpr int ATTN_WARPS = 8;

// STAGE_V: the slice's K and V rows are parked in shared memory (used when the slice fits), and the rows of EARLIER
// positions are requested (cp.async) BEFORE the dependency wait: they were written by launches that finished
// long ago (earlier tokens), so their trip from DRAM overlaps the tail of the kernel in front of this one.  Only the
// newest position's row, written by this kernel (ROPE != 0) or by the rotary kernel right before it (ROPE = 0), is
// fetched after the wait.  *pos is read before the wait for the same reason.
// ROPE: the rotary step of the new token is done here instead of by a kernel of its own.  q is the
// un-rotated query (rotated while it is loaded); the CTA whose slice holds position *pos rotates the new
// key, writes it and the new value into the caches and then reads them back like any other row.
// ROPE = 2: q, k_new, v_new are fixed-point accumulators, rounded to fp16 on read and cleared afterwards (k, v by
// the CTA that consumed them; q by the CTA that merges, i.e. after every CTA of the kv head has read it).
struct RopeArgs {
    void *k_new, *v_new;       // [kv_heads][hd], fp16 (ROPE 1) or fixed-point accumulators (ROPE 2)
    const float *cos_t, *sin_t;  // [max_len][hd / 2]
};
// Sequences decoded in lock step (one shared position): sequence blockIdx.z finds its operands these many BYTES
// further on.  All zero for a single sequence.
struct SeqStrides {
    size_t q, kv_new, cache, out, scratch;
};
template <int ROPE>
__device__ __forceinline__ float rope_in(const void *p, size_t i) {
    if (ROPE == 2) return __half2float(__float2half_rn(acc_value(reinterpret_cast<const acc_t *>(p)[i])));
    return __half2float(reinterpret_cast<const __half *>(p)[i]);
}

// CLUSTER (with STAGE_V, at most 8 slices): the CTAs of a kv head form a thread-block cluster and the slices are merged
// through distributed shared memory — every CTA leaves its partial result in its own shared memory, one cluster
// barrier, CTA 0 of the cluster reads all of them and writes the output, a second barrier keeps the others (and their
// shared memory) alive until it has.  Replaces partials -> fence -> counter -> re-read through L2; no scratch is used.
template <int G, bool STAGE_V, int ROPE, bool CLUSTER = false>
__global__ void __launch_bounds__(ATTN_WARPS * 32) attention_split_kernel(const void *q, __half *k_cache, __half *v_cache,
                                                                          const int64_t *pos_p, __half *out, float *partial,
                                                                          unsigned *counters, int kv_heads, int hd,
                                                                          int max_len, float scale, int nsplit,
                                                                          int slice_cap, RopeArgs ra, SeqStrides ss) {
    extern __shared__ __align__(16) float smem_f[];
    {
        const size_t z = blockIdx.z;
        q = reinterpret_cast<const char *>(q) + z * ss.q;
        ra.k_new = reinterpret_cast<char *>(ra.k_new) + z * ss.kv_new;
        ra.v_new = reinterpret_cast<char *>(ra.v_new) + z * ss.kv_new;
        k_cache = reinterpret_cast<__half *>(reinterpret_cast<char *>(k_cache) + z * ss.cache);
        v_cache = reinterpret_cast<__half *>(reinterpret_cast<char *>(v_cache) + z * ss.cache);
        out = reinterpret_cast<__half *>(reinterpret_cast<char *>(out) + z * ss.out);
        partial = reinterpret_cast<float *>(reinterpret_cast<char *>(partial) + z * ss.scratch);
        counters = reinterpret_cast<unsigned *>(reinterpret_cast<char *>(counters) + z * ss.scratch);
    }
    __shared__ float s_m[G], s_l[G];
    __shared__ float s_w[ATTN_MAX_SPLIT][G];
    __shared__ int s_is_last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int NW = ATTN_WARPS, U = 4;
    float *qf = smem_f;                  // [G][hd], pre-scaled
    float *sc = qf + G * hd;             // [G][slice_cap]
    float *obuf = sc + G * slice_cap;    // [NW][G][hd]
    uint4 *vs = reinterpret_cast<uint4 *>(obuf + NW * G * hd);   // STAGE_V: [slice_cap][hd / 8] 16-byte pieces of the V rows
    uint4 *ks = vs + (size_t)slice_cap * (hd >> 3);              // STAGE_V: the K rows likewise
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int64_t pos = *pos_p;                // written by a launch that finished before this token's launches began
    const bool pos_ok = pos >= 0 && pos < max_len;
    if (pos >= max_len) pos = max_len - 1;
    if (pos < 0) pos = 0;
    const int T = (int)pos + 1;
    const int per = (T + nsplit - 1) / nsplit;
    const int t_begin = split * per;
    const int n = max(0, min(T, t_begin + per) - t_begin);   // positions of this slice (<= slice_cap)
    const int lpr = hd >> 3;             // lanes per row (hd is a power of two: 4, 8, 16 or 32 lanes)
    const int lpr_shift = 31 - __clz(lpr), hd_shift = lpr_shift + 3;
    const int rows = 32 >> lpr_shift;    // positions per warp and load instruction
    const int sub = lane >> lpr_shift, sl = lane & (lpr - 1);
    // the slice that ends with the newest position gets that row after the wait (from this kernel's own rotary step,
    // or from the rotary kernel in front of it); with an out-of-range *pos nothing is written and the row is an old one
    const bool has_newest = n > 0 && t_begin + n == T;
    const bool newest_fresh = has_newest && (ROPE == 0 || pos_ok);
    if (STAGE_V) {
        const int n_old = newest_fresh ? n - 1 : n;
        const size_t stride_h = (size_t)kv_heads * hd;
        const __half *k0 = k_cache + ((size_t)t_begin * kv_heads + kvh) * hd, *v0 = v_cache + ((size_t)t_begin * kv_heads + kvh) * hd;
        for (int idx = tid; idx < n_old * lpr; idx += blockDim.x) {
            const int tl = idx >> lpr_shift, piece = idx & (lpr - 1);
            const size_t off = (size_t)tl * stride_h + piece * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(ks + idx)), "l"(k0 + off) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(vs + idx)), "l"(v0 + off) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (ROPE != 0) {   // the rotary factors of this position: constant tables, asked into L1 ahead of the wait
        const int half = hd >> 1;
        for (int i = tid * 32; i < half; i += blockDim.x * 32) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(ra.cos_t + (size_t)pos * half + i));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(ra.sin_t + (size_t)pos * half + i));
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (ROPE == 0) {
        const __half *qh = reinterpret_cast<const __half *>(q);
        for (int i = tid; i < G * hd; i += blockDim.x) qf[i] = __half2float(qh[(size_t)kvh * G * hd + i]) * scale;
    } else {
        const int half = hd >> 1;
        const float *cs = ra.cos_t + (size_t)pos * half, *sn = ra.sin_t + (size_t)pos * half;
        // One pass over all work items — the G query rotations, and in the CTA whose slice ends with the new token also
        // the key rotation and the value copy — so that the loads of q, k_new and v_new are in flight together instead
        // of one dependent round trip after the other.
        const bool owner = pos_ok && has_newest;
        const int nq = G * half, nk = owner ? half : 0, nv = owner ? hd : 0;
        __half *krow = k_cache + ((size_t)pos * kv_heads + kvh) * hd, *vrow = v_cache + ((size_t)pos * kv_heads + kvh) * hd;
        // STAGE_V: the new row also goes straight to its place among the staged rows
        __half *ksrow = reinterpret_cast<__half *>(ks) + (size_t)(n > 0 ? n - 1 : 0) * hd;
        __half *vsrow = reinterpret_cast<__half *>(vs) + (size_t)(n > 0 ? n - 1 : 0) * hd;
        for (int i = tid; i < nq + nk + nv; i += blockDim.x) {
            if (i < nq) {
                const int g = i >> (hd_shift - 1), j = i & (half - 1);
                const size_t at = ((size_t)kvh * G + g) * hd + j;
                const float a = rope_in<ROPE>(q, at), b = rope_in<ROPE>(q, at + half);
                // rounded to fp16 as a separate rotary kernel would have stored it
                qf[g * hd + j] = __half2float(__float2half_rn(a * cs[j] - b * sn[j])) * scale;
                qf[g * hd + half + j] = __half2float(__float2half_rn(b * cs[j] + a * sn[j])) * scale;
            } else if (i < nq + nk) {
                const int j = i - nq;
                const size_t at = (size_t)kvh * hd + j;
                const float a = rope_in<ROPE>(ra.k_new, at), b = rope_in<ROPE>(ra.k_new, at + half);
                const __half r0 = __float2half_rn(a * cs[j] - b * sn[j]), r1 = __float2half_rn(b * cs[j] + a * sn[j]);
                krow[j] = r0;
                krow[half + j] = r1;
                if (STAGE_V) ksrow[j] = r0, ksrow[half + j] = r1;
            } else {
                const int j = i - nq - nk;
                const __half vn = __float2half_rn(rope_in<ROPE>(ra.v_new, (size_t)kvh * hd + j));
                vrow[j] = vn;
                if (STAGE_V) vsrow[j] = vn;
            }
        }
        if (ROPE == 2 && owner) {   // consumed: cleared for the next token (CTA-uniform branch; all reads above are done)
            __syncthreads();
            for (int j = tid; j < hd; j += blockDim.x) {
                reinterpret_cast<acc_t *>(ra.k_new)[(size_t)kvh * hd + j] = 0;
                reinterpret_cast<acc_t *>(ra.v_new)[(size_t)kvh * hd + j] = 0;
            }
        }
    }
    if (STAGE_V) {
        if (ROPE == 0 && newest_fresh) {   // the row the rotary kernel in front of this one wrote
            const size_t at = ((size_t)pos * kv_heads + kvh) * hd;
            for (int piece = tid; piece < lpr; piece += blockDim.x) {
                ks[(n - 1) * lpr + piece] = *reinterpret_cast<const uint4 *>(k_cache + at + piece * 8);
                vs[(n - 1) * lpr + piece] = *reinterpret_cast<const uint4 *>(v_cache + at + piece * 8);
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    }
    __syncthreads();   // also orders the cache rows written above before this CTA's reads of them
    const size_t row_stride = (size_t)kv_heads * hd;
    const __half *kbase = k_cache + ((size_t)t_begin * kv_heads + kvh) * hd + sl * 8;
    const __half *vbase = v_cache + ((size_t)t_begin * kv_heads + kvh) * hd + sl * 8;
    // ---- scores
    {
        float qr[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int j = 0; j < 8; ++j) qr[g][j] = qf[g * hd + sl * 8 + j];
        for (int base = warp * rows; base < n; base += NW * rows * U) {
            uint4 kk[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int tl = base + u * NW * rows + sub;
                if (STAGE_V) kk[u] = tl < n ? ks[tl * lpr + sl] : make_uint4(0u, 0u, 0u, 0u);
                else kk[u] = tl < n ? *reinterpret_cast<const uint4 *>(kbase + (size_t)tl * row_stride) : make_uint4(0u, 0u, 0u, 0u);
            }
            // all U x G partial dot products first, then the butterfly over the row's lanes on all of them
            // together (independent shuffles pipeline; one value at a time they would serialise on latency)
            float d[U][G];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const __half2 *h = reinterpret_cast<const __half2 *>(&kk[u]);
                float kf[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    kf[2 * j] = f.x;
                    kf[2 * j + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float acc = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc += qr[g][j] * kf[j];
                    d[u][g] = acc;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                if (o < lpr) {
#pragma unroll
                    for (int u = 0; u < U; ++u)
#pragma unroll
                        for (int g = 0; g < G; ++g) d[u][g] += __shfl_xor_sync(0xffffffffu, d[u][g], o);
                }
            }
            if (sl == 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int tl = base + u * NW * rows + sub;
                    if (tl < n) {
#pragma unroll
                        for (int g = 0; g < G; ++g) sc[g * slice_cap + tl] = d[u][g];
                    }
                }
            }
        }
    }
    __syncthreads();
    // ---- slice maximum and sum per query head (one warp per head, round robin)
    for (int g = warp; g < G; g += NW) {
        float m = -INFINITY;
        for (int t = lane; t < n; t += 32) m = fmaxf(m, sc[g * slice_cap + t]);
        m = warp_max(m);
        float l = 0.f;
        for (int t = lane; t < n; t += 32) {
            const float pe = __expf(sc[g * slice_cap + t] - m);
            sc[g * slice_cap + t] = pe;
            l += pe;
        }
        l = warp_sum(l);
        if (lane == 0) {
            s_m[g] = m;
            s_l[g] = l;
        }
    }
    __syncthreads();
    // ---- weighted sum of the V rows
    {
        float o[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int j = 0; j < 8; ++j) o[g][j] = 0.f;
        for (int base = warp * rows; base < n; base += NW * rows * U) {
            uint4 vv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int tl = base + u * NW * rows + sub;
                if (STAGE_V) vv[u] = tl < n ? vs[tl * lpr + sl] : make_uint4(0u, 0u, 0u, 0u);
                else vv[u] = tl < n ? *reinterpret_cast<const uint4 *>(vbase + (size_t)tl * row_stride) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int tl = base + u * NW * rows + sub;
                const __half2 *h = reinterpret_cast<const __half2 *>(&vv[u]);
                float vf[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    vf[2 * j] = f.x;
                    vf[2 * j + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pe = tl < n ? sc[g * slice_cap + tl] : 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[g][j] += pe * vf[j];
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float v = o[g][j];
#pragma unroll
                for (int off = 16; off >= 4; off >>= 1)
                    if (off >= lpr) v += __shfl_xor_sync(0xffffffffu, v, off);
                if (sub == 0) obuf[(warp * G + g) * hd + sl * 8 + j] = v;
            }
    }
    __syncthreads();
    // ---- this slice's result: per query head hd unnormalised outputs, then max and sum
    const int stride = hd + 2;
    if constexpr (CLUSTER) {
        cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();   // (1, nsplit, 1): rank = split
        float *pbuf = reinterpret_cast<float *>(ks + (size_t)slice_cap * lpr);            // [G][hd + 2]
        for (int i = tid; i < G * hd; i += blockDim.x) {
            const int g = i >> hd_shift, d = i & (hd - 1);
            float r = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) r += obuf[(w * G + g) * hd + d];
            pbuf[g * stride + d] = r;
        }
        if (tid < G) {
            pbuf[tid * stride + hd] = s_m[tid];
            pbuf[tid * stride + hd + 1] = s_l[tid];
        }
        cluster.sync();
        if (split == 0) {
            for (int g = warp; g < G; g += NW) {
                float m_sp = -INFINITY, l_sp = 0.f;
                if (lane < nsplit) {
                    const float *ps = cluster.map_shared_rank(pbuf, lane) + g * stride;
                    m_sp = ps[hd];
                    l_sp = ps[hd + 1];
                }
                const float m = warp_max(m_sp);
                const float wgt = lane < nsplit ? __expf(m_sp - m) : 0.f;
                const float l = warp_sum(wgt * l_sp);
                if (lane < nsplit) s_w[lane][g] = wgt / l;
            }
            __syncthreads();
            for (int i = tid; i < G * hd; i += blockDim.x) {
                const int g = i >> hd_shift, d = i & (hd - 1);
                float t[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) t[k] = k < nsplit ? cluster.map_shared_rank(pbuf, k)[g * stride + d] : 0.f;
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) acc += k < nsplit ? s_w[k][g] * t[k] : 0.f;
                out[((size_t)kvh * G + g) * hd + d] = __float2half_rn(acc);
            }
            if (ROPE == 2) {   // every CTA of this kv head has passed the barrier, hence has read the query accumulators
                acc_t *qacc = reinterpret_cast<acc_t *>(const_cast<void *>(q));
                for (int i = tid; i < G * hd; i += blockDim.x) qacc[(size_t)kvh * G * hd + i] = 0;
            }
        }
        cluster.sync();   // nobody leaves while its partial result may still be read
        return;
    }
    float *mine = partial + ((size_t)(kvh * nsplit + split) * G) * stride;
    for (int i = tid; i < G * hd; i += blockDim.x) {
        const int g = i >> hd_shift, d = i & (hd - 1);
        float r = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) r += obuf[(w * G + g) * hd + d];
        __stcg(mine + g * stride + d, r);
    }
    if (tid < G) {
        __stcg(mine + tid * stride + hd, s_m[tid]);
        __stcg(mine + tid * stride + hd + 1, s_l[tid]);
    }
    __syncthreads();
    if (tid == 0) {
        // one acquire-release add per CTA behind the barrier: the release covers the partial results the other threads
        // stored before the barrier, the acquire those of the CTAs that arrived earlier
        unsigned old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(counters + kvh) : "memory");
        s_is_last = (old == (unsigned)(nsplit - 1));
    }
    __syncthreads();
    if (!s_is_last) return;
    const float *all = partial + ((size_t)kvh * nsplit * G) * stride;
    // weight of every slice per query head: exp(slice max - overall max) / overall sum (empty slices: 0)
    // (one warp per query head, lane = slice: all loads of a head are in flight together)
    for (int g = warp; g < G; g += NW) {
        float m_sp = -INFINITY, l_sp = 0.f;
        if (lane < nsplit) {
            const float *ps = all + (size_t)(lane * G + g) * stride;
            m_sp = __ldcg(ps + hd);
            l_sp = __ldcg(ps + hd + 1);
        }
        const float m = warp_max(m_sp);
        const float wgt = lane < nsplit ? __expf(m_sp - m) : 0.f;
        const float l = warp_sum(wgt * l_sp);
        if (lane < nsplit) s_w[lane][g] = wgt / l;
    }
    __syncthreads();
    for (int i = tid; i < G * hd; i += blockDim.x) {
        const int g = i >> hd_shift, d = i & (hd - 1);
        float acc = 0.f;
        for (int s0 = 0; s0 < nsplit; s0 += 8) {
            float t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = (s0 + k < nsplit) ? __ldcg(all + (size_t)((s0 + k) * G + g) * stride + d) : 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) acc += (s0 + k < nsplit) ? s_w[s0 + k][g] * t[k] : 0.f;
        }
        out[((size_t)kvh * G + g) * hd + d] = __float2half_rn(acc);
    }
    if (ROPE == 2) {   // every CTA of this kv head has arrived, hence has read the query accumulators
        acc_t *qacc = reinterpret_cast<acc_t *>(const_cast<void *>(q));
        for (int i = tid; i < G * hd; i += blockDim.x) qacc[(size_t)kvh * G * hd + i] = 0;
    }
    if (tid == 0) counters[kvh] = 0u;   // ready for the next call
}

constexpr size_t ATTN_WS_HEADER = 1024;   // arrival counters, one per kv head (<= 256 heads)

template <int G, bool STAGE_V, int ROPE, bool CLUSTER = false>
int launch_attention_variant(size_t smem, const void *q, const void *k_cache, const void *v_cache, const int64_t *pos, void *out,
                             int kv_heads, int hd, int max_len, float scale, void *workspace, int nsplit, int slice_cap,
                             const RopeArgs &ra, cudaStream_t stream, int batch = 1, const SeqStrides &ss = SeqStrides{}) {
    if (smem + 2048 > 48 * 1024) {   // the kernel's static shared memory counts against the default limit too
        // the attribute belongs to the (function, device) pair: remember it per device ordinal
        static size_t configured[64];
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SAL_E_DEVICE;
        if (configured[dev] < smem) {
            if (cudaFuncSetAttribute(attention_split_kernel<G, STAGE_V, ROPE, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem) != cudaSuccess)
                return SAL_E_LAUNCH;
            configured[dev] = smem;
        }
    }
    if (CLUSTER) {   // the slices of a kv head are one thread-block cluster (at most 8: the portable size)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kv_heads, nsplit, batch);
        cfg.blockDim = dim3(ATTN_WARPS * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 1;
        attr[1].val.clusterDim.y = (unsigned)nsplit;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        {   // once per device and cluster shape: can such a cluster be resident at all?  If not, the caller takes the other merge.
            static signed char fits[64][9];
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || nsplit > 8) return SAL_E_DEVICE;
            if (fits[dev][nsplit] == 0) {
                int clusters = 0;
                const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, attention_split_kernel<G, STAGE_V, ROPE, CLUSTER>, &cfg);
                if (e != cudaSuccess) (void)cudaGetLastError();
                fits[dev][nsplit] = (e == cudaSuccess && clusters >= 1) ? 1 : -1;
            }
            if (fits[dev][nsplit] < 0) return SAL_E_UNSUPPORTED;
        }
        return cudaLaunchKernelEx(&cfg, attention_split_kernel<G, STAGE_V, ROPE, CLUSTER>, q,
                                  reinterpret_cast<__half *>(const_cast<void *>(k_cache)),
                                  reinterpret_cast<__half *>(const_cast<void *>(v_cache)), pos, reinterpret_cast<__half *>(out),
                                  reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + ATTN_WS_HEADER),
                                  reinterpret_cast<unsigned *>(workspace), kv_heads, hd, max_len, scale, nsplit, slice_cap, ra,
                                  ss) == cudaSuccess
                   ? SAL_OK
                   : SAL_E_LAUNCH;
    }
    return launch_pdl(attention_split_kernel<G, STAGE_V, ROPE, CLUSTER>, dim3(kv_heads, nsplit, batch), dim3(ATTN_WARPS * 32), smem, stream, q,
                      reinterpret_cast<__half *>(const_cast<void *>(k_cache)), reinterpret_cast<__half *>(const_cast<void *>(v_cache)),
                      pos, reinterpret_cast<__half *>(out),
                      reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + ATTN_WS_HEADER),
                      reinterpret_cast<unsigned *>(workspace), kv_heads, hd, max_len, scale, nsplit, slice_cap, ra, ss);
}

// Shared memory of one CTA: query, scores, per-warp outputs; staged: K and V rows of a slice; cluster: its partial result.
inline size_t attn_smem_base(int G, int hd, int slice_cap) { return (size_t)(G * hd + G * slice_cap + ATTN_WARPS * G * hd) * sizeof(float); }
inline size_t attn_smem_staged(int G, int hd, int slice_cap) { return attn_smem_base(G, hd, slice_cap) + 2 * (size_t)slice_cap * hd * sizeof(__half); }
inline size_t attn_smem_cluster(int G, int hd, int slice_cap) { return attn_smem_staged(G, hd, slice_cap) + (size_t)G * (hd + 2) * sizeof(float); }
constexpr size_t ATTN_CLUSTER_SMEM_MAX = 160 * 1024;

template <int G, int ROPE>
int launch_attention_split(const void *q, const void *k_cache, const void *v_cache, const int64_t *pos, void *out, int kv_heads,
                           int hd, int max_len, float scale, void *workspace, int nsplit, int slice_cap, const RopeArgs &ra,
                           cudaStream_t stream, int batch = 1, const SeqStrides &ss = SeqStrides{}, bool cluster = false) {
    const size_t base = attn_smem_base(G, hd, slice_cap);
    const size_t staged = attn_smem_staged(G, hd, slice_cap);
    if (cluster) {   // the caller has checked that the staged rows fit
        const int rc = launch_attention_variant<G, true, ROPE, true>(attn_smem_cluster(G, hd, slice_cap), q, k_cache, v_cache, pos, out,
                                                                     kv_heads, hd, max_len, scale, workspace, nsplit, slice_cap, ra, stream,
                                                                     batch, ss);
        if (rc != SAL_E_UNSUPPORTED) return rc;   // unsupported: no such cluster can be resident here; merge through L2 instead
    }
    if (staged <= 96 * 1024)
        return launch_attention_variant<G, true, ROPE>(staged, q, k_cache, v_cache, pos, out, kv_heads, hd, max_len, scale,
                                                       workspace, nsplit, slice_cap, ra, stream, batch, ss);
    if (base > 200 * 1024) return SAL_E_UNSUPPORTED;
    return launch_attention_variant<G, false, ROPE>(base, q, k_cache, v_cache, pos, out, kv_heads, hd, max_len, scale, workspace,
                                                    nsplit, slice_cap, ra, stream, batch, ss);
}

template <int ROPE>
int attention_split_entry(const void *q, const void *k_cache, const void *v_cache, const int64_t *pos, void *out, int heads,
                          int kv_heads, int hd, int max_len, float scale, void *workspace, size_t workspace_bytes,
                          const RopeArgs &ra, void *stream, int batch = 1) {
    if (!q || !k_cache || !v_cache || !pos || !out || !workspace) return SAL_E_NULL;
    if (batch < 1 || batch > 64) return SAL_E_SHAPE;
    if (heads < 1 || kv_heads < 1 || kv_heads > 256 || heads % kv_heads || max_len < 1 || max_len > 65536) return SAL_E_SHAPE;
    if (hd != 32 && hd != 64 && hd != 128 && hd != 256) return SAL_E_UNSUPPORTED;
    const size_t ws_seq = ATTN_WS_HEADER + (size_t)heads * ATTN_MAX_SPLIT * (size_t)(hd + 2) * sizeof(float);   // per sequence
    if (workspace_bytes < ws_seq * (size_t)batch) return SAL_E_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) return SAL_E_ALIGN;
    const int G = heads / kv_heads;
    // about three CTAs per SM (they are small), at least ~16 positions per slice at the longest context
    int nsplit = (444 + kv_heads * batch - 1) / (kv_heads * batch);
    if (nsplit > ATTN_MAX_SPLIT) nsplit = ATTN_MAX_SPLIT;
    if (G >= 8 && nsplit > ATTN_MAX_SPLIT / 2) nsplit = ATTN_MAX_SPLIT / 2;   // the merge grows with G x slices (measured)
    if (nsplit > (max_len + 15) / 16) nsplit = (max_len + 15) / 16;
    if (nsplit < 1) nsplit = 1;
    // capacity of a slice, rounded up to a multiple of 4: the staged V rows behind the G x slice_cap scores in
    // shared memory are written with 16-byte stores
    int slice_cap = ((max_len + nsplit - 1) / nsplit + 3) & ~3;
    // Up to 8 slices whose K and V rows fit into shared memory: the slices of a kv head run as one thread-block
    // cluster and are merged through distributed shared memory (longer contexts keep the merge through L2).
    bool cluster = false;
    if (nsplit > 1) {
        // about 160 CTAs in all (measured on 32 kv heads x 600 positions: 4 to 6 slices beat 8 and 3; on 8 kv heads of
        // 8 query heads x 1100 positions: 8 beat 6 and 4), the rows being in flight before the dependency wait anyway
        int ns_c = (160 + kv_heads * batch - 1) / (kv_heads * batch);
        if (ns_c > 8) ns_c = 8;
        if (ns_c < 2) ns_c = 2;
        if (ns_c > nsplit) ns_c = nsplit;
        const int cap_c = ((max_len + ns_c - 1) / ns_c + 3) & ~3;
        if (attn_smem_cluster(heads / kv_heads, hd, cap_c) <= ATTN_CLUSTER_SMEM_MAX) {
            cluster = true;
            nsplit = ns_c;
            slice_cap = cap_c;
        }
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // sequences in lock step: operands of sequence z lie z rows / caches / scratch blocks further on
    const size_t qelem = ROPE == 2 ? sizeof(acc_t) : sizeof(__half);
    SeqStrides ss = {};
    if (batch > 1) {
        ss.q = (size_t)heads * hd * qelem;
        ss.kv_new = (size_t)kv_heads * hd * qelem;
        ss.cache = (size_t)max_len * kv_heads * hd * sizeof(__half);
        ss.out = (size_t)heads * hd * sizeof(__half);
        ss.scratch = ws_seq;
    }
    switch (G) {
        case 1: return launch_attention_split<1, ROPE>(q, k_cache, v_cache, pos, out, kv_heads, hd, max_len, scale, workspace, nsplit, slice_cap, ra, s, batch, ss, cluster);
        case 2: return launch_attention_split<2, ROPE>(q, k_cache, v_cache, pos, out, kv_heads, hd, max_len, scale, workspace, nsplit, slice_cap, ra, s, batch, ss, cluster);
        case 4: return launch_attention_split<4, ROPE>(q, k_cache, v_cache, pos, out, kv_heads, hd, max_len, scale, workspace, nsplit, slice_cap, ra, s, batch, ss, cluster);
        case 8: return launch_attention_split<8, ROPE>(q, k_cache, v_cache, pos, out, kv_heads, hd, max_len, scale, workspace, nsplit, slice_cap, ra, s, batch, ss, cluster);
        default: return SAL_E_UNSUPPORTED;
    }
}

}  // namespace

extern "C" {

int sal_residual_rmsnorm_f16(const void *x, const void *delta, const void *weight, void *out, void *x_out, int n, float eps,
                             void *stream) {
    if (!x || !weight || !out) return SAL_E_NULL;
    if (n < 1 || n > 12000 /* the row is staged in shared memory, 48 KB with the reduction scratch */) return SAL_E_SHAPE;
    const int threads = n >= 1024 ? 1024 : ((n + 31) / 32) * 32;
    return launch_pdl(residual_rmsnorm_kernel, dim3(1), dim3(threads), (size_t)n * sizeof(float), stream,
                      reinterpret_cast<const __half *>(x), reinterpret_cast<const __half *>(delta),
                      reinterpret_cast<const __half *>(weight), reinterpret_cast<__half *>(out),
                      reinterpret_cast<__half *>(x_out), n, eps);
}

int sal_rope_kv_write_f16(void *q, const void *k, const void *v, const void *cos, const void *sin, const int64_t *pos,
                          void *k_cache, void *v_cache, int heads, int kv_heads, int hd, int max_len, void *stream) {
    if (!q || !k || !v || !cos || !sin || !pos || !k_cache || !v_cache) return SAL_E_NULL;
    if (heads < 1 || kv_heads < 1 || hd < 2 || (hd & 1) || max_len < 1) return SAL_E_SHAPE;
    const int total = heads * (hd / 2) + kv_heads * (hd / 2) + kv_heads * hd;
    return launch_pdl(rope_kv_write_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, reinterpret_cast<__half *>(q),
                      reinterpret_cast<const __half *>(k), reinterpret_cast<const __half *>(v),
                      reinterpret_cast<const float *>(cos), reinterpret_cast<const float *>(sin), pos,
                      reinterpret_cast<__half *>(k_cache), reinterpret_cast<__half *>(v_cache), heads, kv_heads, hd, max_len);
}

int sal_residual_rmsnorm_fixedacc(const void *x, void *delta_acc, const void *weight, void *out, void *x_out, int n, float eps,
                                void *zero_a, int zero_a_n, void *zero_b, int zero_b_n, void *stream) {
    if (!x || !weight || !out) return SAL_E_NULL;
    if (n < 1 || n > 12000 /* the row is staged in shared memory, 48 KB with the reduction scratch */ || zero_a_n < 0 || zero_b_n < 0 || (zero_a_n && !zero_a) || (zero_b_n && !zero_b)) return SAL_E_SHAPE;
    const int threads = n >= 1024 ? 1024 : ((n + 31) / 32) * 32;
    // one CTA for the norm, plus one per 16 K extra accumulator words to clear (at most 32)
    int zero_ctas = (zero_a_n + zero_b_n + 16383) / 16384;
    if (zero_ctas > 32) zero_ctas = 32;
    return launch_pdl(residual_rmsnorm_acc_kernel, dim3(1 + zero_ctas), dim3(threads), (size_t)n * sizeof(float), stream,
                      reinterpret_cast<const __half *>(x), reinterpret_cast<acc_t *>(delta_acc),
                      reinterpret_cast<const __half *>(weight), reinterpret_cast<__half *>(out), reinterpret_cast<__half *>(x_out),
                      n, eps, reinterpret_cast<acc_t *>(zero_a), zero_a_n, reinterpret_cast<acc_t *>(zero_b), zero_b_n);
}

int sal_rope_kv_write_fixedacc(void *q_acc, void *k_acc, void *v_acc, void *q_out, const void *cos, const void *sin,
                             const int64_t *pos, void *k_cache, void *v_cache, int heads, int kv_heads, int hd, int max_len,
                             void *stream) {
    if (!q_acc || !k_acc || !v_acc || !q_out || !cos || !sin || !pos || !k_cache || !v_cache) return SAL_E_NULL;
    if (heads < 1 || kv_heads < 1 || hd < 2 || (hd & 1) || max_len < 1) return SAL_E_SHAPE;
    const int total = heads * (hd / 2) + kv_heads * (hd / 2) + kv_heads * hd;
    return launch_pdl(rope_kv_write_acc_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, reinterpret_cast<acc_t *>(q_acc),
                      reinterpret_cast<acc_t *>(k_acc), reinterpret_cast<acc_t *>(v_acc), reinterpret_cast<__half *>(q_out),
                      reinterpret_cast<const float *>(cos), reinterpret_cast<const float *>(sin), pos,
                      reinterpret_cast<__half *>(k_cache), reinterpret_cast<__half *>(v_cache), heads, kv_heads, hd, max_len);
}

int sal_attention_decode_f16(const void *q, const void *k_cache, const void *v_cache, const int64_t *pos, void *out, int heads,
                             int kv_heads, int hd, int max_len, float scale, void *stream) {
    if (!q || !k_cache || !v_cache || !pos || !out) return SAL_E_NULL;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads || hd < 2 || hd > 256 || (hd & 1) || max_len < 1 || max_len > 16384)
        return SAL_E_SHAPE;
    const size_t smem = (size_t)(hd + max_len + 32 * hd) * sizeof(float);
    if (smem > 48 * 1024) {
        static bool configured[64];   // per device ordinal: the attribute is not shared between devices
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SAL_E_DEVICE;
        if (!configured[dev]) {
            if (cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024) != cudaSuccess)
                return SAL_E_LAUNCH;
            configured[dev] = true;
        }
    }
    return launch_pdl(attention_decode_kernel, dim3(heads), dim3(1024), smem, stream, reinterpret_cast<const __half *>(q),
                      reinterpret_cast<const __half *>(k_cache), reinterpret_cast<const __half *>(v_cache), pos,
                      reinterpret_cast<__half *>(out), heads, kv_heads, hd, max_len, scale);
}

size_t sal_attention_workspace_bytes(int heads, int hd) {
    if (heads < 1 || hd < 1) return 0;
    return ATTN_WS_HEADER + (size_t)heads * ATTN_MAX_SPLIT * (size_t)(hd + 2) * sizeof(float);
}

int sal_attention_decode_split_f16(const void *q, const void *k_cache, const void *v_cache, const int64_t *pos, void *out,
                                   int heads, int kv_heads, int hd, int max_len, float scale, void *workspace,
                                   size_t workspace_bytes, void *stream) {
    return attention_split_entry<0>(q, k_cache, v_cache, pos, out, heads, kv_heads, hd, max_len, scale, workspace, workspace_bytes,
                                    RopeArgs{}, stream);
}

int sal_rope_attention_decode(void *q, void *k_new, void *v_new, int inputs_fixed, const void *cos, const void *sin,
                              const int64_t *pos, void *k_cache, void *v_cache, void *out, int heads, int kv_heads, int hd,
                              int max_len, float scale, void *workspace, size_t workspace_bytes, void *stream) {
    if (!k_new || !v_new || !cos || !sin) return SAL_E_NULL;
    const RopeArgs ra = {k_new, v_new, reinterpret_cast<const float *>(cos), reinterpret_cast<const float *>(sin)};
    return inputs_fixed ? attention_split_entry<2>(q, k_cache, v_cache, pos, out, heads, kv_heads, hd, max_len, scale, workspace,
                                                 workspace_bytes, ra, stream)
                      : attention_split_entry<1>(q, k_cache, v_cache, pos, out, heads, kv_heads, hd, max_len, scale, workspace,
                                                 workspace_bytes, ra, stream);
}

int sal_rope_attention_decode_batch(void *q, void *k_new, void *v_new, const void *cos, const void *sin, const int64_t *pos,
                                    void *k_cache, void *v_cache, void *out, int batch, int heads, int kv_heads, int hd, int max_len,
                                    float scale, void *workspace, size_t workspace_bytes, void *stream) {
    if (!k_new || !v_new || !cos || !sin) return SAL_E_NULL;
    const RopeArgs ra = {k_new, v_new, reinterpret_cast<const float *>(cos), reinterpret_cast<const float *>(sin)};
    return attention_split_entry<1>(q, k_cache, v_cache, pos, out, heads, kv_heads, hd, max_len, scale, workspace, workspace_bytes, ra,
                                    stream, batch);
}

int sal_residual_rmsnorm_rows_f16(const void *x, const void *delta, const void *weight, void *out, void *x_out, int rows, int n,
                                  float eps, void *stream) {
    if (!x || !weight || !out) return SAL_E_NULL;
    if (rows < 1 || rows > 65535 || n < 1 || n > 12000) return SAL_E_SHAPE;
    const int threads = n >= 1024 ? 1024 : ((n + 31) / 32) * 32;
    return launch_pdl(residual_rmsnorm_kernel, dim3(rows), dim3(threads), (size_t)n * sizeof(float), stream,
                      reinterpret_cast<const __half *>(x), reinterpret_cast<const __half *>(delta), reinterpret_cast<const __half *>(weight),
                      reinterpret_cast<__half *>(out), reinterpret_cast<__half *>(x_out), n, eps);
}

int sal_greedy_token_f16(const void *logits_f16, void *logits_f32, int vocab, int64_t *token, int64_t *pos, void *stream) {
    if (!logits_f16 || !token || !pos) return SAL_E_NULL;
    if (vocab < 8 || vocab % 8 != 0) return SAL_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(logits_f16) & 15) || (reinterpret_cast<uintptr_t>(logits_f32) & 15)) return SAL_E_ALIGN;
    return launch_pdl(greedy_token_kernel, dim3(1), dim3(1024), 0, stream, reinterpret_cast<const __half *>(logits_f16),
                      reinterpret_cast<float *>(logits_f32), vocab, token, pos);
}

int sal_silu_mul_f16(const void *gate, const void *up, void *out, int n, void *stream) {
    if (!gate || !up || !out) return SAL_E_NULL;
    if (n < 1) return SAL_E_SHAPE;
    return launch_pdl(silu_mul_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, reinterpret_cast<const __half *>(gate),
                      reinterpret_cast<const __half *>(up), reinterpret_cast<__half *>(out), n);
}

}  // extern "C"
