/*
 * sal_decode_ops.h — the element-wise / attention steps that sit between the BCQ LUT-GEMV calls
 * of a batch-1 LLaMA-architecture decode step (same shared library as sal_lutgemm.h).
 *
 * The reference leaves these steps to Hugging Face's decoder layer: it only swaps the nn.Linear
 * modules named in model/llama.py:93-98 (q/k/v/o/gate/up/down) and times the unmodified model
 * (model/opt.py:366-423).  They are provided here fused, so that a decoded token costs a dozen
 * launches per block instead of ~45.  All pointers are device pointers; `pos` is a DEVICE int64
 * holding the current position, so the calls are CUDA-graph capturable with a moving position.
 * Return values: SAL_OK or a negative SAL_E_* code (see sal_lutgemm.h).
 */
#ifndef SAL_DECODE_OPS_H
#define SAL_DECODE_OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* t = x (+ delta if delta != NULL); if x_out != NULL, x_out = t (the updated residual stream);
 * out = t * rsqrt(mean(t^2) + eps) * weight.  fp16 tensors of n elements, fp32 arithmetic.
 * x_out may alias x.  1 <= n <= 12000. */
int sal_residual_rmsnorm_f16(const void *x, const void *delta, const void *weight, void *out, void *x_out, int n,
                             float eps, void *stream);

/* Rotary embedding (rotate-half convention) of q [heads][hd] in place and of k [kv_heads][hd] into
 * k_cache[*pos], plus v [kv_heads][hd] into v_cache[*pos].  Caches: fp16 [max_len][kv_heads][hd].
 * cos/sin: fp32 [max_len][hd/2]. */
int sal_rope_kv_write_f16(void *q, const void *k, const void *v, const void *cos, const void *sin, const int64_t *pos,
                          void *k_cache, void *v_cache, int heads, int kv_heads, int hd, int max_len, void *stream);

/* Variants for products that ran with SAL_OUT_FIXED_ATOMIC (their outputs are 64-bit fixed-point accumulators,
 * signed integers in units of 2**-32, see include/sal_lutgemm.h).  Every
 * accumulator element is rounded to fp16 when read — the value the fp16-output path would have stored — and
 * then set back to zero, so the buffer is ready for the same layer's product of the next token.
 * sal_residual_rmsnorm_fixedacc: as sal_residual_rmsnorm_f16 with delta an accumulator vector (may be NULL); additionally clears
 * zero_a[0..zero_a_n) and zero_b[0..zero_b_n) (accumulators, e.g. gate and up, whose reader was a GEMV).
 * sal_rope_kv_write_fixedacc: as sal_rope_kv_write_f16 with q, k, v accumulator vectors; the rotated query goes to q_out (fp16). */
int sal_residual_rmsnorm_fixedacc(const void *x, void *delta_acc, const void *weight, void *out, void *x_out, int n,
                                float eps, void *zero_a, int zero_a_n, void *zero_b, int zero_b_n, void *stream);
int sal_rope_kv_write_fixedacc(void *q_acc, void *k_acc, void *v_acc, void *q_out, const void *cos, const void *sin,
                             const int64_t *pos, void *k_cache, void *v_cache, int heads, int kv_heads, int hd,
                             int max_len, void *stream);

/* Single-query attention over cache positions 0..*pos: out [heads][hd] fp16.  Grouped-query
 * attention when heads > kv_heads (heads % kv_heads == 0).  hd <= 256, max_len <= 16384. */
int sal_attention_decode_f16(const void *q, const void *k_cache, const void *v_cache, const int64_t *pos, void *out,
                             int heads, int kv_heads, int hd, int max_len, float scale, void *stream);

/* The same attention split over the cached positions (kv_heads x up to 32 CTAs instead of one CTA per head;
 * a K / V row is read once for all query heads of its group).  Where the K and V rows of a slice fit into
 * shared memory (up to 8 slices), the slices of a kv head run as one thread-block cluster and are merged through
 * distributed shared memory; longer contexts are merged through the scratch buffer by the last CTA of a kv head to
 * finish.  hd in {32, 64, 128, 256}, heads / kv_heads in {1, 2, 4, 8}, caches 16-byte aligned;
 * other shapes return SAL_E_UNSUPPORTED (use sal_attention_decode_f16).  `workspace`: caller-owned scratch of
 * sal_attention_workspace_bytes(heads, hd) bytes, zero-filled once (arrival counters reset themselves), not
 * shared between streams.
 * Ordering contract of the split kernels (this one, sal_rope_attention_decode and its batch form): they are
 * launched with programmatic dependent launch and read *pos and the cache rows of positions BEFORE *pos ahead of
 * their dependency wait, so that those rows are already on their way while the kernel in front drains.  These
 * must therefore be complete when the launch DIRECTLY in front of this one starts — true whenever they were
 * written by an earlier token's launches and the token boundary holds at least one ordinary (fully serialising)
 * launch or a synchronisation, as any sampler does.  Row *pos itself, q and k_new / v_new are read after the wait. */
size_t sal_attention_workspace_bytes(int heads, int hd);
int sal_attention_decode_split_f16(const void *q, const void *k_cache, const void *v_cache, const int64_t *pos, void *out,
                                   int heads, int kv_heads, int hd, int max_len, float scale, void *workspace,
                                   size_t workspace_bytes, void *stream);

/* Rotary step + cache write + split attention in ONE kernel (one launch less per decoder block).  q [heads][hd],
 * k_new / v_new [kv_heads][hd] are the un-rotated projections of the new token: fp16 (inputs_fixed = 0; q is
 * left as it is), or fixed-point accumulators (inputs_fixed = 1) that are rounded to fp16 on read and cleared.  The
 * rotated key and the value are stored at position *pos of the caches (nothing is stored if *pos is outside
 * 0..max_len-1) and attention runs over positions 0..*pos.  Same shape limits, scratch buffer and results as
 * sal_rope_kv_write_f16 followed by sal_attention_decode_split_f16. */
int sal_rope_attention_decode(void *q, void *k_new, void *v_new, int inputs_fixed, const void *cos, const void *sin,
                              const int64_t *pos, void *k_cache, void *v_cache, void *out, int heads, int kv_heads, int hd,
                              int max_len, float scale, void *workspace, size_t workspace_bytes, void *stream);

/* The two helpers above for `batch` sequences decoded in lock step (one shared position *pos; 1 <= batch <= 64), so
 * that a lock-step batch decoder has no framework operator between its small-batch LUT products either.
 * sal_residual_rmsnorm_rows_f16: `rows` rows of n elements (x, delta, out, x_out are [rows][n]; one weight vector).
 * sal_rope_attention_decode_batch: q [batch][heads][hd], k_new / v_new [batch][kv_heads][hd] (fp16, un-rotated),
 * caches [batch][max_len][kv_heads][hd], out [batch][heads][hd]; scratch of batch x
 * sal_attention_workspace_bytes(heads, hd) bytes, zero-filled once.  Per sequence exactly what
 * sal_rope_attention_decode computes. */
int sal_residual_rmsnorm_rows_f16(const void *x, const void *delta, const void *weight, void *out, void *x_out, int rows, int n,
                                  float eps, void *stream);
int sal_rope_attention_decode_batch(void *q, void *k_new, void *v_new, const void *cos, const void *sin, const int64_t *pos,
                                    void *k_cache, void *v_cache, void *out, int batch, int heads, int kv_heads, int hd, int max_len,
                                    float scale, void *workspace, size_t workspace_bytes, void *stream);

/* End of a greedy decode step in one launch: logits_f16 [vocab] (as an fp16 lm_head product leaves them) are copied
 * to logits_f32 (may be NULL), *token = index of the largest logit (the smallest index among equal maxima, as
 * torch.argmax; NaNs are never selected) and *pos += 1.  Replaces the convert / copy / argmax / copy / add
 * operators a framework runs there.  vocab % 8 == 0, logits_f16 16-byte aligned. */
int sal_greedy_token_f16(const void *logits_f16, void *logits_f32, int vocab, int64_t *token, int64_t *pos, void *stream);

/* out = silu(gate) * up, fp16 vectors of n elements. */
int sal_silu_mul_f16(const void *gate, const void *up, void *out, int n, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SAL_DECODE_OPS_H */
