// Thin extern "C" shim over the reference's OWN host code, compiled from the reference's
// headers where they lie (include path given on the command line by oracle/Makefile; no
// reference source is copied here).  TEST INFRASTRUCTURE ONLY: it validates the C
// restatement in mgv_oracle.c, generates the golden fixtures, and is the timed
// "reference" CPU baseline.  Built against CUTLASS 4.5.0 headers (the reference pins
// 3.4.1, which is not available offline).
//
// The reference reports errors by printing and calling exit(-1); a shim called from a
// test process must not die, so every precondition the reference checks is checked
// here first and turned into a negative return code.

#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "cutlass/numeric_types.h"
#include "cutlass/half.h"

#include "utils/type_base.h"

namespace host {
// The reference's interleave template for W8_A16 needs a 64-bit access type that
// utils/type_base.h:55-61 does not provide; supplying it is the only addition.
template <>
struct AccessTypeDeduce<64> {
  using type = int64_t;
};
}  // namespace host

#include "utils/preprocess.h"
#include "utils/vector_subbyte.h"
#include "host/mixed_gemv.h"

using half_t = cutlass::half_t;
using HostGemv = host::reference::MixedGemv<cutlass::int4b_t, half_t, half_t, int8_t, half_t,
                                            float, float>;

extern "C" {

int ref_pack_int4(int8_t *packed, const int8_t *unpacked, size_t n_unpacked) {
  host::utils::SubBytePacker<cutlass::int4b_t, int8_t>::pack(packed, unpacked, n_unpacked);
  return 0;
}

int ref_unpack_int4(int8_t *unpacked, const int8_t *packed, size_t n_packed) {
  host::utils::SubBytePacker<cutlass::int4b_t, int8_t>::unpack(unpacked, packed, n_packed);
  return 0;
}

int ref_preprocess_zeros(uint16_t *dst, const uint16_t *scales, const int8_t *zeros, int n) {
  host::utils::ZeroPointPreprocessor<half_t, int8_t>::neg_zero_point_multiplies_scale(
      reinterpret_cast<half_t *>(dst), reinterpret_cast<const half_t *>(scales), zeros, n);
  return 0;
}

// MixedGemvWeightPreprocessor::run for W4_A16; for W8_A16 the same three steps through
// the reference's own templates (its public dispatcher refuses W8_A16).
int ref_preprocess_weights(int8_t *dst, const int8_t *src, const size_t *shape, int rank,
                           int layout, int quant_type) {
  if (rank != 2 && rank != 3) return -1;
  if (quant_type != int(host::QuantType::W4_A16) && quant_type != int(host::QuantType::W8_A16))
    return -2;
  const int bits = quant_type == int(host::QuantType::W4_A16) ? 4 : 8;
  const size_t K = shape[rank - 2], N = shape[rank - 1];
  if (layout == int(host::LayoutType::kRowMajor) && ((N * bits / 8) % 32 || (K * bits / 8) % 32))
    return -3;
  if (N % size_t(16 / bits)) return -4;
  if (K % 8) return -5;
  std::vector<size_t> shp(shape, shape + rank);
  if (bits == 4) {
    host::utils::MixedGemvWeightPreprocessor::run(dst, src, shp, host::LayoutType(layout),
                                                  host::QuantType::W4_A16, false);
    return 0;
  }
  size_t n_bytes = 1;
  for (size_t d : shp) n_bytes *= d;
  std::vector<int8_t> a(src, src + n_bytes), b(n_bytes);
  if (layout == int(host::LayoutType::kRowMajor)) {
    host::utils::SubbyteWeightProcessor::subbyte_transpose(b.data(), a.data(), shp,
                                                           host::QuantType::W8_A16);
    a.swap(b);
  }
  std::swap(shp[rank - 1], shp[rank - 2]);
  host::utils::SubbyteWeightProcessor::interleave_row_major_tensor_impl<host::QuantType::W8_A16>(
      b.data(), a.data(), shp);
  host::utils::SubbyteWeightProcessor::add_bias_and_interleave_quantized_tensor_inplace(
      b.data(), n_bytes, host::QuantType::W8_A16);
  std::memcpy(dst, b.data(), n_bytes);
  return 0;
}

// host::reference::MixedGemv::operator() on rows [0, N) of an int4 matrix.
//   w_packed  un-preprocessed nibbles, element (n,k) at n*K+k
//   zero      int8 [G][N] (all zero when the mode has none)
static void run_rows(int N, int K, int group, const uint8_t *w_packed, const uint16_t *x,
                     const uint16_t *scale, const int8_t *zero, const uint16_t *bias,
                     uint16_t *out) {
  host::utils::vector_subbyte<cutlass::int4b_t> A(size_t(N) * K, cutlass::int4b_t(0));
  std::memcpy(A.raw_data(), w_packed, size_t(N) * K / 2);
  HostGemv op;
  op(1, N, 1, K, group, A, reinterpret_cast<const half_t *>(x),
     reinterpret_cast<const half_t *>(scale), zero, reinterpret_cast<const half_t *>(bias),
     reinterpret_cast<half_t *>(out));
}

int ref_host_gemv_int4(int N, int K, int group, const uint8_t *w_packed, const uint16_t *x,
                       const uint16_t *scale, const int8_t *zero, const uint16_t *bias,
                       uint16_t *out, int n_threads) {
  if (group <= 0 || K % group || (size_t(N) * K) % 2) return -1;
  if (n_threads <= 1) {
    run_rows(N, K, group, w_packed, x, scale, zero, bias, out);
    return 0;
  }
  // The reference loop has no threading; rows are independent, so the unmodified
  // operator() is run on disjoint row ranges, each with its own [G][rows] scale slice.
  const int G = K / group;
  std::vector<std::thread> pool;
  const int rows_per = ((N + n_threads - 1) / n_threads + 1) & ~1;  // even: whole bytes
  for (int n0 = 0; n0 < N; n0 += rows_per) {
    const int rows = std::min(rows_per, N - n0);
    pool.emplace_back([=]() {
      std::vector<uint16_t> s(size_t(G) * rows);
      std::vector<int8_t> z(size_t(G) * rows);
      for (int g = 0; g < G; ++g)
        for (int r = 0; r < rows; ++r) {
          s[size_t(g) * rows + r] = scale[size_t(g) * N + n0 + r];
          z[size_t(g) * rows + r] = zero[size_t(g) * N + n0 + r];
        }
      run_rows(rows, K, group, w_packed + size_t(n0) * K / 2, x, s.data(), z.data(),
               bias ? bias + n0 : nullptr, out + n0);
    });
  }
  for (auto &t : pool) t.join();
  return 0;
}

int ref_hardware_threads() { return int(std::thread::hardware_concurrency()); }

}  // extern "C"
