/*
 * C ABI of the load-time packers: +-1 planes -> packed 32-bit words, and the published
 * "Lat." checkpoint layout -> the layout the LUT-GEMV kernels read.  Device pointers,
 * sizes, a cudaStream_t passed as void*; returns SAL_OK or a negative SAL_E_* code
 * (sal_lutgemm.h).  Integer work: results are bit-exact with the reference's Python.
 */
#ifndef SAL_PACK_H_
#define SAL_PACK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Replaces pack_binaryWeight (lut_gemm/kernel.py:9-23), the step the reference leaves on the
 * CPU ("TODO: perform packing on GPU", model/opt.py:287).
 *   signs: int8 [R][C][q], +1 or -1 (the reference's [R, n_groups, group_size, wbit] flattened);
 *          C % 32 == 0.
 *   out:   int32, bit t of word j of row r, plane b = (signs[r][32 j + t][b] == +1);
 *          kernel_layout = 0: [R][C/32][q] (what pack_binaryWeight returns),
 *          kernel_layout = 1: [C/32][q][R] (what the kernels read: permute(1, 2, 0) of the former).
 *   bad:   optional int32 counter (may be NULL), incremented for every element that is neither
 *          +1 nor -1 (the reference asserts on such input).
 */
int sal_pack_planes_i8(const void *signs, void *out, int R, int C, int q, int kernel_layout, int *bad, void *stream);

/*
 * Replaces convert_weight (lut_gemm/kernel.py:112-133) for any shape (the reference's version
 * only works for square layers): the checkpoint tensor is packed along OUTPUT features,
 *   in:  int32 [K][N/32][q], bit t of word j of row k = plane bit of (input k, output 32 j + t),
 * the kernels want it packed along INPUT features,
 *   out: int32 [K/32][q][N], bit t of word kk, plane b, column n = bit of (input 32 kk + t, output n).
 * K % 32 == 0, N % 32 == 0.
 */
int sal_repack_lat_to_kernel(const void *in, void *out, int K, int N, int q, void *stream);

#ifdef __cplusplus
}
#endif
#endif
