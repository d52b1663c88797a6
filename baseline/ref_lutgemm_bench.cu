// Timing harness around the REFERENCE's own CUDA kernel for the mode-A product (M = 1):
// nqmv_bias_shift_mulq -> _nqmv_bias_shift_mulq<32> (lut_gemm/mv_fp16_bias.hpp:498-579, 766-774), the
// kernel behind lutgemm_compute_shift_scale.  The header is NOT part of this repository: it is included
// from the reference tree at build time (-I <reference>/lut_gemm, see build_ref_gpu.py) and compiled
// unmodified for sm_100a.  The result is an informational comparator ("how fast is the kernel this
// project replaces on the same GPU"); the benchmark's reference arm stays the CPU path.
//
// Prints one JSON line: per LLaMA-2-7B shape (3 bit, g128) the microseconds per call over a rotation of
// weight copies larger than L2 (CUDA events on the legacy default stream, which is where the reference
// launches), GB/s of the same algorithmic bytes bench.py counts, and a correctness check of a small case
// against a host computation (fp16 atomics: tolerance 3e-2 of max|y|).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "mv_fp16_bias.hpp"

#define CK(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_));            \
            return 2;                                                                     \
        }                                                                                 \
    } while (0)

static uint64_t g_state = 0x9E3779B97F4A7C15ull;
static uint32_t next_u32() {  // splitmix64
    uint64_t z = (g_state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (uint32_t)((z ^ (z >> 31)) >> 16);
}

__global__ void fill_words(uint32_t *p, size_t n, uint32_t seed) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t v = (uint32_t)i * 2654435761u + seed;
        v ^= v >> 15; v *= 2246822519u; v ^= v >> 13; v *= 3266489917u; v ^= v >> 16;
        p[i] = v;
    }
}
__global__ void fill_alpha(__half *p, size_t n, uint32_t seed) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t v = (uint32_t)i * 2246822519u + seed;
        v ^= v >> 15; v *= 2654435761u; v ^= v >> 13;
        p[i] = __float2half(exp2f(-(float)(2 + v % 7)));   // 2**-k, k in 2..8
    }
}

static int check_small(double *err_out) {
    const int K = 512, N = 256, Q = 3, G = 128;
    std::vector<uint32_t> w((size_t)(K / 32) * Q * N);
    std::vector<__half> alpha((size_t)(K / G) * Q * N), x(K);
    for (auto &v : w) v = next_u32() ^ (next_u32() << 16);
    for (auto &v : alpha) v = __float2half(exp2f(-(float)(2 + next_u32() % 7)));
    for (auto &v : x) v = __float2half(((int)(next_u32() % 2001) - 1000) / 1000.0f);
    std::vector<double> ref(N, 0.0);
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
            for (int b = 0; b < Q; ++b) {
                const int bit = (w[((size_t)(k / 32) * Q + b) * N + n] >> (k % 32)) & 1;
                ref[n] += (double)__half2float(alpha[((size_t)(k / G) * Q + b) * N + n]) * (bit ? 1.0 : -1.0) * __half2float(x[k]);
            }
    uint32_t *dw; __half *da, *dx, *dy;
    CK(cudaMalloc(&dw, w.size() * 4)); CK(cudaMalloc(&da, alpha.size() * 2)); CK(cudaMalloc(&dx, K * 2)); CK(cudaMalloc(&dy, N * 2));
    CK(cudaMemcpy(dw, w.data(), w.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(da, alpha.data(), alpha.size() * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dx, x.data(), K * 2, cudaMemcpyHostToDevice));
    CK(cudaMemset(dy, 0, N * 2));
    nqmv_bias_shift_mulq(dy, dw, da, N, K, Q, K / G, dx, 0);
    CK(cudaGetLastError());
    CK(cudaDeviceSynchronize());
    std::vector<__half> y(N);
    CK(cudaMemcpy(y.data(), dy, N * 2, cudaMemcpyDeviceToHost));
    double num = 0, den = 0;
    for (int n = 0; n < N; ++n) {
        num = fmax(num, fabs((double)__half2float(y[n]) - ref[n]));
        den = fmax(den, fabs(ref[n]));
    }
    *err_out = num / (den > 0 ? den : 1);
    cudaFree(dw); cudaFree(da); cudaFree(dx); cudaFree(dy);
    return 0;
}

int main() {
    double err = 0;
    if (int rc = check_small(&err)) return rc;
    if (!(err <= 3e-2)) {
        fprintf(stderr, "reference kernel fails its small check: max relative error %g\n", err);
        return 3;
    }
    const int Q = 3, G = 128;
    const int shapes[3][2] = {{4096, 4096}, {4096, 11008}, {11008, 4096}};
    const int per_block[3] = {4, 2, 1};   // products of each shape in one decoder block
    double us[3], block_us = 0, block_bytes = 0;
    char rows[1024];
    size_t off = 0;
    for (int s = 0; s < 3; ++s) {
        const int K = shapes[s][0], N = shapes[s][1];
        const size_t words = (size_t)(K / 32) * Q * N, alphas = (size_t)(K / G) * Q * N;
        int copies = (int)(((size_t)320 << 20) / (words * 4)) + 1;   // rotation larger than the 126 MB L2
        if (copies < 4) copies = 4;
        std::vector<uint32_t *> dw(copies);
        __half *da, *dx, *dy;
        for (int c = 0; c < copies; ++c) {
            CK(cudaMalloc(&dw[c], words * 4));
            fill_words<<<1184, 256>>>(dw[c], words, 17u + 101u * c + 7u * s);
        }
        CK(cudaMalloc(&da, alphas * 2)); CK(cudaMalloc(&dx, K * 2)); CK(cudaMalloc(&dy, N * 2));
        fill_alpha<<<1184, 256>>>(da, alphas, 5u + s);
        std::vector<__half> x(K);
        for (auto &v : x) v = __float2half(((int)(next_u32() % 2001) - 1000) / 4000.0f);
        CK(cudaMemcpy(dx, x.data(), K * 2, cudaMemcpyHostToDevice));
        CK(cudaMemset(dy, 0, N * 2));
        CK(cudaDeviceSynchronize());
        for (int c = 0; c < copies; ++c) nqmv_bias_shift_mulq(dy, dw[c], da, N, K, Q, K / G, dx, 0);   // warm-up pass
        CK(cudaGetLastError());
        CK(cudaDeviceSynchronize());
        cudaEvent_t e0, e1;
        CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
        const int reps = 5;
        CK(cudaMemset(dy, 0, N * 2));
        CK(cudaEventRecord(e0, 0));
        for (int r = 0; r < reps; ++r)
            for (int c = 0; c < copies; ++c) nqmv_bias_shift_mulq(dy, dw[c], da, N, K, Q, K / G, dx, 0);
        CK(cudaEventRecord(e1, 0));
        CK(cudaEventSynchronize(e1));
        CK(cudaGetLastError());
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, e0, e1));
        us[s] = ms * 1e3 / (reps * copies);
        const double bytes = (double)K * N * Q / 8 + (double)(K / G) * N * Q * 2 + 2.0 * K;
        block_us += per_block[s] * us[s];
        block_bytes += per_block[s] * bytes;
        off += snprintf(rows + off, sizeof(rows) - off, "%s{\"K\": %d, \"N\": %d, \"us_per_call\": %.3f, \"gbps\": %.1f}", s ? ", " : "", K, N,
                        us[s], bytes / us[s] / 1e3);
        for (int c = 0; c < copies; ++c) cudaFree(dw[c]);
        cudaFree(da); cudaFree(dx); cudaFree(dy);
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    printf("{\"kernel\": \"reference nqmv_bias_shift_mulq (lut_gemm/mv_fp16_bias.hpp:498-579), unmodified, built for sm_100a\", "
           "\"workload\": \"LLaMA-2-7B shapes, M=1, 3-bit g128, one launch per product on the legacy default stream, weights rotated beyond L2\", "
           "\"shapes\": [%s], \"decoder_block_us\": %.2f, \"value\": %.1f, \"unit\": \"GB/s\", \"small_check_max_rel_err\": %.4g}\n",
           rows, block_us, block_bytes / block_us / 1e3, err);
    return 0;
}
