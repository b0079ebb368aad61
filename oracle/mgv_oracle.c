/*
 * CPU oracle (test infrastructure; see mgv_oracle.h for scope and parity status).
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: the reference accumulates with a separate fp32 multiply
 * and add (host/mixed_gemv.h:98), not a fused one.
 */
#include "mgv_oracle.h"

#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- fp16 <-> fp32, round to nearest even (cutlass::half_t host conversion) ---- */

float mgv_oracle_h2f(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int shift = 0;
      while (!(man & 0x400u)) {
        man <<= 1;
        ++shift;
      }
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t mgv_oracle_f2h(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  uint32_t a = x & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((a > 0x7F800000u) ? 0x200u : 0));
  }
  if (a >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (a < 0x33000001u) { /* <= 2^-25: rounds to zero (ties to even -> 0) */
    return sign;
  }
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
  int shift;                                /* bits dropped from m */
  uint32_t base;
  if (e >= -14) {
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    m &= 0x7FFFFFu; /* implicit bit is carried by the exponent field */
  } else {
    shift = 13 + (-14 - e); /* subnormal half: keep the implicit bit */
    base = 0;
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q; /* carry may roll into the exponent: intended */
  return (uint16_t)(sign | (base + q));
}

static inline uint16_t h_mul(uint16_t a, uint16_t b) {
  return mgv_oracle_f2h(mgv_oracle_h2f(a) * mgv_oracle_h2f(b));
}
static inline uint16_t h_add(uint16_t a, uint16_t b) {
  return mgv_oracle_f2h(mgv_oracle_h2f(a) + mgv_oracle_h2f(b));
}
static inline uint16_t h_neg(uint16_t a) { return (uint16_t)(a ^ 0x8000u); }

/* ---- a1: nibble packing, utils/preprocess.h:41-84 ---- */

void mgv_oracle_pack_int4(uint8_t *packed, const int8_t *unpacked, size_t n_unpacked) {
  for (size_t i = 0; i < n_unpacked / 2; ++i) {
    uint8_t lo = (uint8_t)unpacked[2 * i] & 0x0F;
    uint8_t hi = (uint8_t)((uint8_t)unpacked[2 * i + 1] << 4);
    packed[i] = (uint8_t)(lo | hi);
  }
}

static inline int sext4(unsigned v) { return (int)((v & 0xF) ^ 8) - 8; }

void mgv_oracle_unpack_int4(int8_t *unpacked, const uint8_t *packed, size_t n_packed) {
  for (size_t i = 0; i < n_packed; ++i) {
    unpacked[2 * i] = (int8_t)sext4(packed[i]);
    unpacked[2 * i + 1] = (int8_t)sext4(packed[i] >> 4);
  }
}

/* ---- a2: [rows, cols] -> [cols, rows] on packed elements, utils/preprocess.h:123-268 ---- */

static inline unsigned get_elt(const uint8_t *p, size_t idx, int bits) {
  if (bits == 8) return p[idx];
  return (p[idx >> 1] >> (4 * (idx & 1))) & 0xF;
}
static inline void set_elt(uint8_t *p, size_t idx, int bits, unsigned v) {
  if (bits == 8) {
    p[idx] = (uint8_t)v;
  } else {
    unsigned sh = 4 * (idx & 1);
    p[idx >> 1] = (uint8_t)((p[idx >> 1] & ~(0xFu << sh)) | ((v & 0xF) << sh));
  }
}

static int transpose_packed(uint8_t *dst, const uint8_t *src, size_t experts, size_t rows,
                            size_t cols, int bits) {
  /* the reference insists on 32-byte multiples in both directions (:151-162) */
  if ((cols * bits / 8) % 32 || (rows * bits / 8) % 32) return -3;
  size_t mat_bytes = rows * cols * bits / 8;
  for (size_t e = 0; e < experts; ++e) {
    const uint8_t *s = src + e * mat_bytes;
    uint8_t *d = dst + e * mat_bytes;
    for (size_t r = 0; r < rows; ++r)
      for (size_t c = 0; c < cols; ++c) set_elt(d, c * rows + r, bits, get_elt(s, r * cols + c, bits));
  }
  return 0;
}

/* ---- a3: row interleave at 8-element granularity, utils/preprocess.h:292-348 ----
 * interleave factor = 16 / bits rows (4 for int4, 2 for int8); one access = 8 elements. */

static int interleave_rows(uint8_t *dst, const uint8_t *src, size_t experts, size_t rows,
                           size_t cols, int bits) {
  size_t il = 16 / bits;
  size_t acc_bytes = 8 * bits / 8; /* bytes in one 8-element access */
  if (rows % il) return -4;
  if (cols % 8) return -5;
  size_t acc_per_row = cols / 8;
  for (size_t e = 0; e < experts; ++e) {
    size_t base = e * rows * acc_per_row;
    for (size_t r = 0; r < rows; ++r)
      for (size_t c = 0; c < acc_per_row; ++c) {
        size_t in = base + r * acc_per_row + c;
        size_t out = base + (r / il) * (acc_per_row * il) + c * il + (r % il);
        memcpy(dst + out * acc_bytes, src + in * acc_bytes, acc_bytes);
      }
  }
  return 0;
}

/* ---- a4: +8 and nibble permutation per 32-bit word, utils/preprocess.h:393-455 ---- */

static int bias_permute_int4(uint8_t *p, size_t n_elts) {
  if (n_elts % 8) return -6;
  size_t n_words = n_elts / 8;
  for (size_t w = 0; w < n_words; ++w) {
    uint32_t in = (uint32_t)p[4 * w] | ((uint32_t)p[4 * w + 1] << 8) |
                  ((uint32_t)p[4 * w + 2] << 16) | ((uint32_t)p[4 * w + 3] << 24);
    uint32_t out = 0;
    for (int d = 0; d < 8; ++d) {
      int s = d < 4 ? 2 * d : 2 * (d - 4) + 1; /* :446 */
      uint32_t v = (uint32_t)(sext4(in >> (4 * s)) + 8) & 0xF;
      out |= v << (4 * d);
    }
    p[4 * w] = (uint8_t)out;
    p[4 * w + 1] = (uint8_t)(out >> 8);
    p[4 * w + 2] = (uint8_t)(out >> 16);
    p[4 * w + 3] = (uint8_t)(out >> 24);
  }
  return 0;
}

/* ---- a5: +128 and swap of bytes 1 and 2 in every four, utils/preprocess.h:365-391 ---- */

static int bias_permute_int8(uint8_t *p, size_t n_elts) {
  if (n_elts % 4) return -7;
  for (size_t i = 0; i < n_elts; ++i) p[i] = (uint8_t)(p[i] + 128);
  for (size_t b = 0; b < n_elts; b += 4) {
    uint8_t t = p[b + 1];
    p[b + 1] = p[b + 2];
    p[b + 2] = t;
  }
  return 0;
}

/* ---- a6: MixedGemvWeightPreprocessor::run, utils/preprocess.h:480-522 ---- */

int mgv_oracle_preprocess_weights(uint8_t *dst, const uint8_t *src, const size_t *shape,
                                  int rank, int layout, int quant_type) {
  if (rank != 2 && rank != 3) return -1;
  int bits;
  if (quant_type == MGV_O_W8_A16)
    bits = 8;
  else if (quant_type == MGV_O_W4_A16)
    bits = 4;
  else
    return -2; /* W4_AFP8 is refused by the interleave dispatcher (:353-361) */
  size_t experts = rank == 3 ? shape[0] : 1;
  size_t K = shape[rank - 2], N = shape[rank - 1];
  size_t n_elts = experts * K * N;
  size_t n_bytes = n_elts * bits / 8;
  uint8_t *a = (uint8_t *)malloc(n_bytes ? n_bytes : 1);
  uint8_t *b = (uint8_t *)malloc(n_bytes ? n_bytes : 1);
  if (!a || !b) {
    free(a);
    free(b);
    return -8;
  }
  memcpy(a, src, n_bytes);
  int rc = 0;
  if (layout == MGV_O_ROW_MAJOR) { /* [K,N] with N contiguous -> [N,K] (:505-511) */
    rc = transpose_packed(b, a, experts, K, N, bits);
    uint8_t *t = a;
    a = b;
    b = t;
  }
  if (!rc) rc = interleave_rows(b, a, experts, N, K, bits); /* :517 on the swapped shape */
  if (!rc) rc = bits == 4 ? bias_permute_int4(b, n_elts) : bias_permute_int8(b, n_elts);
  if (!rc) memcpy(dst, b, n_bytes);
  free(a);
  free(b);
  return rc;
}

/* ---- a7: utils/preprocess.h:94-101 ---- */

void mgv_oracle_preprocess_zeros(uint16_t *dst, const uint16_t *scales, const int8_t *zeros,
                                 size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = h_mul(mgv_oracle_f2h((float)(-(int)zeros[i])), scales[i]);
}

/* ---- a19: host/mixed_gemv.h:82-104 ---- */

int mgv_oracle_gemv(int M, int N, int K, int bits, int group_size, const uint8_t *w,
                    const uint16_t *x, int64_t ldx, const uint16_t *scale, const void *zero,
                    int zero_kind, const uint16_t *bias, float alpha, float beta,
                    uint16_t *out, int64_t ldd, float *out_f32, int n_threads) {
  if (bits != 4 && bits != 8) return -1;
  if (group_size <= 0 || K % group_size) return -2;
  if (zero_kind != MGV_O_ZERO_NONE && !zero) return -3;
  const int8_t *zero_i8 = (const int8_t *)zero;
  const uint16_t *zero_h = (const uint16_t *)zero;
  if (n_threads < 1) n_threads = 1;
#ifdef _OPENMP
#pragma omp parallel for num_threads(n_threads) schedule(static)
#endif
  for (int n = 0; n < N; ++n) {
    for (int m = 0; m < M; ++m) {
      float acc = 0.0f; /* :84 */
      for (int k = 0; k < K; ++k) {
        int g = k / group_size; /* :88 */
        size_t idx = (size_t)n * K + k;
        int q = bits == 4 ? sext4(get_elt(w, idx, 4)) : (int)(int8_t)w[idx];
        uint16_t s = scale[(size_t)g * N + n];
        uint16_t dq = h_mul(mgv_oracle_f2h((float)q), s); /* half(q) * scale, :95-96 */
        if (zero_kind == MGV_O_ZERO_INT8) {
          /* -(scale * half(zero)), :92-93 */
          uint16_t sxz = h_neg(h_mul(s, mgv_oracle_f2h((float)zero_i8[(size_t)g * N + n])));
          dq = h_add(dq, sxz);
        } else if (zero_kind == MGV_O_ZERO_F16) {
          dq = h_add(dq, zero_h[(size_t)g * N + n]);
        }
        acc += mgv_oracle_h2f(x[(size_t)m * ldx + k]) * mgv_oracle_h2f(dq); /* :98 */
      }
      if (out_f32) out_f32[(size_t)m * ldd + n] = acc;
      if (out) {
        /* :102-103 with the device epilogue's alpha/beta (epilogue/threadblock/epilogue.h:78-97) */
        float b = bias ? mgv_oracle_h2f(bias[n]) : 0.0f; /* bias_val is 0 when absent, :102 */
        float v = alpha * acc;
        v = v + beta * b;
        out[(size_t)m * ldd + n] = mgv_oracle_f2h(v);
      }
    }
  }
  return 0;
}

/* ---- layout contract read-back ---- */

int mgv_oracle_read_preprocessed(const uint8_t *pre, int N, int K, int bits, int n, int k) {
  (void)N;
  if (bits == 4) {
    size_t word = (size_t)(n / 4) * ((size_t)K / 8 * 4) + (size_t)(k / 8) * 4 + (size_t)(n % 4);
    int s = k % 8;
    int d = (s % 2 == 0) ? s / 2 : 4 + (s - 1) / 2;
    uint32_t v = (uint32_t)pre[4 * word] | ((uint32_t)pre[4 * word + 1] << 8) |
                 ((uint32_t)pre[4 * word + 2] << 16) | ((uint32_t)pre[4 * word + 3] << 24);
    return (int)((v >> (4 * d)) & 0xF) - 8;
  }
  size_t unit = (size_t)(n / 2) * ((size_t)K / 8 * 2) + (size_t)(k / 8) * 2 + (size_t)(n % 2);
  int b = k % 8, wd = b / 4, t = b % 4;
  int tp = t == 1 ? 2 : (t == 2 ? 1 : t);
  return (int)pre[unit * 8 + (size_t)wd * 4 + tp] - 128;
}

int mgv_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
