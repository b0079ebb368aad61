/*
 * CPU oracle for the weight-only-quantised GEMV path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA library and the timed CPU baseline of the benchmark.
 * Nothing in the shipped package may call it; the product path has no CPU fallback.
 *
 * Every function restates, in plain C, one piece of the reference's host code and
 * names the reference file:line it follows.  fp16 values travel as uint16_t bit
 * patterns; every fp16 operation is "convert to float, operate, round to nearest
 * even back to fp16", which is what cutlass::half_t does on the host.
 *
 * Parity status:
 *   int4 weights, int8 zero-points, bias       pinned: compared bit-for-bit with the
 *                                              reference's own host code (oracle/_ref)
 *                                              and with fixtures generated from it.
 *   int8 weight preprocessing                  pinned at template level only (the
 *                                              reference's public entry refuses W8_A16).
 *   int8-weight GEMV, fp16 additive zeros,     parity unpinned: the reference has no
 *   batch M > 1, alpha/beta                    host code for them; the loop below is the
 *                                              int4 loop with the one operand swapped.
 */
#ifndef MGV_ORACLE_H_
#define MGV_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* utils/type_base.h:7-16 */
enum { MGV_O_W8_A16 = 0, MGV_O_W4_A16 = 1, MGV_O_W4_AFP8 = 2 };
enum { MGV_O_ROW_MAJOR = 0, MGV_O_COLUMN_MAJOR = 1 };

/* how the zero operand of mgv_oracle_gemv is given */
enum {
  MGV_O_ZERO_NONE = 0, /* no zero term                                              */
  MGV_O_ZERO_INT8 = 1, /* int8 zero-points, host/mixed_gemv.h:92-93                  */
  MGV_O_ZERO_F16 = 2   /* fp16 additive term, already -zero*scale (device format)    */
};

uint16_t mgv_oracle_f2h(float f);
float mgv_oracle_h2f(uint16_t h);

/* utils/preprocess.h:55-84 / :41-53 */
void mgv_oracle_pack_int4(uint8_t *packed, const int8_t *unpacked, size_t n_unpacked);
void mgv_oracle_unpack_int4(int8_t *unpacked, const uint8_t *packed, size_t n_packed);

/* utils/preprocess.h:480-522.  shape = {K,N} (rank 2) or {E,K,N} (rank 3).
 * Returns 0, or a negative code where the reference would print and exit. */
int mgv_oracle_preprocess_weights(uint8_t *dst, const uint8_t *src, const size_t *shape,
                                  int rank, int layout, int quant_type);

/* utils/preprocess.h:94-101 */
void mgv_oracle_preprocess_zeros(uint16_t *dst, const uint16_t *scales, const int8_t *zeros,
                                 size_t n);

/* host/mixed_gemv.h:82-104, generalised over weight width, zero format and batch.
 *   w          un-preprocessed weights, element (n,k) at linear index n*K+k:
 *              bits==4 -> packed nibbles (even index low), bits==8 -> int8 bytes
 *   x          fp16 [M][ldx]
 *   scale      fp16 [G][N], G = K/group_size
 *   zero       per zero_kind: int8 [G][N] or fp16 [G][N] or NULL
 *   bias       fp16 [N] or NULL
 *   out        fp16 [M][ldd];  out = half(alpha*acc + beta*bias)
 *   out_f32    optional float [M][ldd] receiving the fp32 accumulator before the epilogue
 *   n_threads  rows are split over this many OpenMP threads (1 = the reference's loop)
 */
int mgv_oracle_gemv(int M, int N, int K, int bits, int group_size, const uint8_t *w,
                    const uint16_t *x, int64_t ldx, const uint16_t *scale, const void *zero,
                    int zero_kind, const uint16_t *bias, float alpha, float beta,
                    uint16_t *out, int64_t ldd, float *out_f32, int n_threads);

/* Inverse of the preprocessing, used to check the layout contract the device
 * converters rely on (gemv/interleaved_numeric_conversion.h:55-88, :225-298):
 * signed weight (n,k) read back from a preprocessed buffer of a {K,N} matrix. */
int mgv_oracle_read_preprocessed(const uint8_t *pre, int N, int K, int bits, int n, int k);

int mgv_oracle_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
