// Load-time packers (see include/sal_pack.h): HBM-bound bit shuffling, one pass over the data.
#include <cuda_runtime.h>
#include <stdint.h>

#include "sal_lutgemm.h"
#include "sal_pack.h"

namespace {

// One thread per (32-element word, row): reads the 32 x q sign bytes of its word (contiguous in
// memory) with 16-byte loads where alignment allows and writes q words.  Threads of a warp take
// consecutive rows, so the kernel-layout stores ([C/32][q][R]) are coalesced.
template <bool KERNEL_LAYOUT>
__global__ void __launch_bounds__(256) pack_planes_kernel(const int8_t *__restrict__ signs, uint32_t *__restrict__ out, int R,
                                                          int C, int q, int *bad) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    const int j = blockIdx.y;
    if (r >= R) return;
    const int8_t *src = signs + ((size_t)r * C + (size_t)j * 32) * q;
    uint32_t words[SAL_MAX_Q];
#pragma unroll
    for (int b = 0; b < SAL_MAX_Q; ++b) words[b] = 0u;
    int n_bad = 0;
    const int total = 32 * q;   // bytes of this word, element-major then plane
    const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && (total % 16 == 0);
    int t = 0, b = 0;           // element and plane of the next byte
    const auto take = [&](int8_t v) {
        if (v == 1) {
#pragma unroll
            for (int bb = 0; bb < SAL_MAX_Q; ++bb)
                if (bb == b) words[bb] |= 1u << t;
        } else if (v != -1) {
            ++n_bad;
        }
        if (++b == q) {
            b = 0;
            ++t;
        }
    };
    if (vec) {
        for (int i = 0; i < total; i += 16) {
            const int4 chunk = *reinterpret_cast<const int4 *>(src + i);
            const int8_t *c8 = reinterpret_cast<const int8_t *>(&chunk);
#pragma unroll
            for (int k = 0; k < 16; ++k) take(c8[k]);
        }
    } else {
        for (int i = 0; i < total; ++i) take(src[i]);
    }
    const int words_per_row = C / 32;
    for (int bb = 0; bb < q; ++bb) {
        uint32_t w = 0;
#pragma unroll
        for (int k = 0; k < SAL_MAX_Q; ++k)
            if (k == bb) w = words[k];
        if (KERNEL_LAYOUT) out[((size_t)j * q + bb) * R + r] = w;
        else out[((size_t)r * words_per_row + j) * q + bb] = w;
    }
    if (n_bad && bad) atomicAdd(bad, n_bad);
}

// Bit transpose of 32 x 32 tiles.  A CTA stages 32 input rows x TJ words x q planes in shared memory
// with coalesced loads (a row of the checkpoint tensor is contiguous), then each warp takes tiles
// (word j, plane b): lane t holds the word of input row 32 kk + t, and 32 ballots turn the tile
// around; lane i keeps the word of output column 32 j + i.
constexpr int TJ = 32;
__global__ void __launch_bounds__(256) repack_lat_kernel(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, int K,
                                                         int N, int q) {
    extern __shared__ uint32_t tile[];   // [32 rows][TJ * q (+1 pad)]
    const int kk = blockIdx.x, j0 = blockIdx.y * TJ;
    const int nw = N / 32;
    const int tj = min(TJ, nw - j0);
    const int row_words = tj * q, pitch = TJ * q + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int rrow = warp; rrow < 32; rrow += 8) {
        const uint32_t *src = in + ((size_t)(32 * kk + rrow) * nw + j0) * q;
        for (int c = lane; c < row_words; c += 32) tile[rrow * pitch + c] = src[c];
    }
    __syncthreads();
    for (int item = warp; item < tj * q; item += 8) {   // item = (word j, plane b) in the order they are stored
        const int jl = item / q, b = item % q;
        const uint32_t w = tile[lane * pitch + item];
        uint32_t mine = 0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const uint32_t col = __ballot_sync(0xffffffffu, (w >> i) & 1u);
            if (lane == i) mine = col;
        }
        out[((size_t)kk * q + b) * N + (size_t)(j0 + jl) * 32 + lane] = mine;
    }
}

}  // namespace

extern "C" {

int sal_pack_planes_i8(const void *signs, void *out, int R, int C, int q, int kernel_layout, int *bad, void *stream) {
    if (!signs || !out) return SAL_E_NULL;
    if (R < 1 || C < 32 || C % 32 || q < 1 || q > SAL_MAX_Q || C / 32 > 65535) return SAL_E_SHAPE;
    const dim3 grid((unsigned)((R + 255) / 256), (unsigned)(C / 32));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (kernel_layout)
        pack_planes_kernel<true><<<grid, 256, 0, s>>>(reinterpret_cast<const int8_t *>(signs), reinterpret_cast<uint32_t *>(out), R,
                                                      C, q, bad);
    else
        pack_planes_kernel<false><<<grid, 256, 0, s>>>(reinterpret_cast<const int8_t *>(signs), reinterpret_cast<uint32_t *>(out), R,
                                                       C, q, bad);
    return cudaGetLastError() == cudaSuccess ? SAL_OK : SAL_E_LAUNCH;
}

int sal_repack_lat_to_kernel(const void *in, void *out, int K, int N, int q, void *stream) {
    if (!in || !out) return SAL_E_NULL;
    if (K < 32 || K % 32 || N < 32 || N % 32 || q < 1 || q > SAL_MAX_Q) return SAL_E_SHAPE;
    const int nw = N / 32;
    if ((nw + TJ - 1) / TJ > 65535) return SAL_E_SHAPE;
    const dim3 grid((unsigned)(K / 32), (unsigned)((nw + TJ - 1) / TJ));
    const size_t smem = (size_t)32 * (TJ * q + 1) * sizeof(uint32_t);
    repack_lat_kernel<<<grid, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint32_t *>(in),
                                                                                   reinterpret_cast<uint32_t *>(out), K, N, q);
    return cudaGetLastError() == cudaSuccess ? SAL_OK : SAL_E_LAUNCH;
}

}  // extern "C"
