// GPU weight / zero-point preparation.  One pass over the weights replaces the reference's
// host pipeline (utils/preprocess.h:480-522): optional transpose, row interleave, signed ->
// unsigned bias and the in-word element permutation.  Output is bit-exact with the host code.
//
// Output layout (little-endian 32-bit words), signed weight v = W[n][k]:
//   4 bit: word (n/4)*(K/8*4) + (k/8)*4 + n%4 holds k = 8c..8c+7 of row n; nibble d holds
//          element s = (d < 4 ? 2d : 2(d-4)+1), stored as v+8.        (:338-345, :399-454)
//   8 bit: 8-byte unit (n/2)*(K/8*2) + (k/8)*2 + n%2; inside each 4 bytes the elements sit in
//          order e0 e2 e1 e3, stored as v+128.                        (:338-345, :367-390)
// HBM-bound byte shuffling.  Three kernels: the general one below stages a 64x64-element tile in
// shared memory element by element (any shape the interface admits); preprocess_direct_kernel
// serves K-contiguous input without shared memory; preprocess_transpose4_kernel serves 4-bit
// N-contiguous input word by word.  All three produce the same bytes.
#include <algorithm>

#include "mgv_common.cuh"

namespace mgv {
namespace {

constexpr int kTile = 64;      // elements per tile edge
constexpr int kThreads = 256;

// tile[n_local][k_local] holds the biased unsigned value of one element.
template <int BITS, bool ROW_MAJOR_IN>
__global__ void __launch_bounds__(kThreads)
preprocess_weights_kernel(uint32_t *__restrict__ dst, const uint32_t *__restrict__ src, int K, int N) {
  __shared__ uint8_t tile[kTile][kTile + 4];
  constexpr int EPW = 32 / BITS;                 // elements per 32-bit word: 8 or 4
  constexpr int WPR = kTile / EPW;               // words per tile row: 8 or 16
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  constexpr uint32_t BIAS = 1u << (BITS - 1);    // +8 / +128 on a two's-complement field = xor
  const int k0 = blockIdx.x * kTile, n0 = blockIdx.y * kTile;
  const size_t mat_words = size_t(K) * N / EPW;
  src += size_t(blockIdx.z) * mat_words;
  dst += size_t(blockIdx.z) * mat_words;

  // ---- load: 64 rows of WPR words, consecutive threads on consecutive words ----
  for (int i = threadIdx.x; i < kTile * WPR; i += kThreads) {
    const int row = i / WPR, wcol = i % WPR;
    uint32_t word = 0;
    if (!ROW_MAJOR_IN) {  // row = n, the word covers EPW consecutive k
      const int n = n0 + row, k = k0 + wcol * EPW;
      if (n < N && k < K) word = __ldg(src + (size_t(n) * K + k) / EPW);
#pragma unroll
      for (int e = 0; e < EPW; ++e)
        tile[row][wcol * EPW + e] = uint8_t(((word >> (BITS * e)) & MASK) ^ BIAS);
    } else {              // row = k, the word covers EPW consecutive n
      const int k = k0 + row, n = n0 + wcol * EPW;
      if (k < K && n < N) word = __ldg(src + (size_t(k) * N + n) / EPW);
#pragma unroll
      for (int e = 0; e < EPW; ++e)
        tile[wcol * EPW + e][row] = uint8_t(((word >> (BITS * e)) & MASK) ^ BIAS);
    }
  }
  __syncthreads();

  // ---- store: one output word per thread-iteration, consecutive threads on consecutive words ----
  if (BITS == 4) {
    // tile = 16 row-blocks x 8 chunks x 4 rows
    for (int i = threadIdx.x; i < 16 * 8 * 4; i += kThreads) {
      const int j = i & 3, c = (i >> 2) & 7, rb = i >> 5;
      const int nl = 4 * rb + j, n = n0 + nl, k = k0 + 8 * c;
      if (n >= N || k >= K) continue;
      uint32_t out = 0;
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        const int s = d < 4 ? 2 * d : 2 * (d - 4) + 1;
        out |= uint32_t(tile[nl][8 * c + s]) << (4 * d);
      }
      dst[size_t(n / 4) * (size_t(K) / 8 * 4) + size_t(k / 8) * 4 + j] = out;
    }
  } else {
    // tile = 32 row-pairs x 8 chunks x 2 rows x 2 words
    for (int i = threadIdx.x; i < 32 * 8 * 2 * 2; i += kThreads) {
      const int w = i & 1, j = (i >> 1) & 1, c = (i >> 2) & 7, rp = i >> 5;
      const int nl = 2 * rp + j, n = n0 + nl, k = k0 + 8 * c;
      if (n >= N || k >= K) continue;
      const uint8_t *e = &tile[nl][8 * c + 4 * w];
      const uint32_t out = uint32_t(e[0]) | (uint32_t(e[2]) << 8) | (uint32_t(e[1]) << 16) |
                           (uint32_t(e[3]) << 24);
      dst[(size_t(n / 2) * (size_t(K) / 8 * 2) + size_t(k / 8) * 2 + j) * 2 + w] = out;
    }
  }
}

// ---- the common case without a transpose: K-contiguous input, K a multiple of 32 (4 bit) or 16
// (8 bit), 16-byte aligned buffers.  No shared memory: a thread takes one 16-byte piece of each
// row of a row group (4 rows x 32 k, or 2 rows x 16 k), so a warp reads 512 contiguous bytes per
// row and writes 2 KB (1 KB) contiguous; bias and in-word permutation are a few logic operations
// per word.  Bit-exact with the tile kernel above.

// one 4-bit word: +8 on every nibble, then elements 0,2,4,6 to nibbles 0..3 and 1,3,5,7 to 4..7
__device__ __forceinline__ uint32_t permute_w4(uint32_t w) {
  w ^= 0x88888888u;
  uint32_t ev = w & 0x0f0f0f0fu, od = (w >> 4) & 0x0f0f0f0fu;
  ev = (ev | (ev >> 4)) & 0x00ff00ffu;
  ev = (ev | (ev >> 8)) & 0x0000ffffu;
  od = (od | (od >> 4)) & 0x00ff00ffu;
  od = (od | (od >> 8)) & 0x0000ffffu;
  return ev | (od << 16);
}
// one 8-bit word: +128 on every byte, then elements 1 and 2 swapped
__device__ __forceinline__ uint32_t permute_w8(uint32_t w) { return __byte_perm(w ^ 0x80808080u, 0u, 0x3120); }

template <int BITS>
__global__ void __launch_bounds__(256) preprocess_direct_kernel(uint4 *__restrict__ dst, const uint4 *__restrict__ src, size_t K,
                                                                size_t groups, size_t pieces_per_row) {
  constexpr int RPG = 16 / BITS;  // rows per group: 4 or 2
  const size_t total = groups * pieces_per_row;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t grp = i / pieces_per_row, piece = i - grp * pieces_per_row;
    uint4 in[RPG];
#pragma unroll
    for (int r = 0; r < RPG; ++r) in[r] = __ldcs(src + (grp * RPG + r) * pieces_per_row + piece);
    uint4 *out = dst + grp * (RPG * pieces_per_row) + piece * RPG;  // the group's K-major run of 16-byte units
    if constexpr (BITS == 4) {
      // piece = 4 words = 4 chunks of 8 k; unit of chunk c = {row0, row1, row2, row3} word c
      const uint32_t w[4][4] = {{in[0].x, in[0].y, in[0].z, in[0].w}, {in[1].x, in[1].y, in[1].z, in[1].w},
                                {in[2].x, in[2].y, in[2].z, in[2].w}, {in[3].x, in[3].y, in[3].z, in[3].w}};
#pragma unroll
      for (int c = 0; c < 4; ++c)
        __stcs(out + c, make_uint4(permute_w4(w[0][c]), permute_w4(w[1][c]), permute_w4(w[2][c]), permute_w4(w[3][c])));
    } else {
      // piece = 16 k = 2 chunks of 8 k (2 words each); unit of chunk c = {row0 two words, row1 two words}
      __stcs(out + 0, make_uint4(permute_w8(in[0].x), permute_w8(in[0].y), permute_w8(in[1].x), permute_w8(in[1].y)));
      __stcs(out + 1, make_uint4(permute_w8(in[0].z), permute_w8(in[0].w), permute_w8(in[1].z), permute_w8(in[1].w)));
    }
  }
}

// ---- 4-bit weights from N-contiguous input (the layout the reference transposes on the host,
// utils/preprocess.h:123-180), K a multiple of 64.  A block takes 64 k x 256 n: the load is 64 rows
// of 128 contiguous bytes, word for word into shared memory (rows 33 words apart); every thread
// then builds whole 16-byte units -- 4 rows x 8 k -- from eight of those words with byte permutes
// and masks, and eight neighbouring threads write the 128 contiguous bytes of one row group (a 128-k tile measured slower).
__device__ __forceinline__ uint32_t squeeze_low_nibbles(uint32_t v) {  // one nibble per byte -> 16 bits
  v = (v | (v >> 4)) & 0x00ff00ffu;
  return (v | (v >> 8)) & 0x0000ffffu;
}

__global__ void __launch_bounds__(256) preprocess_transpose4_kernel(uint4 *__restrict__ dst, const uint32_t *__restrict__ src, int K, int N) {
  constexpr int TK = 64, TN = 256, PITCH = 33;
  __shared__ uint32_t tile[TK * PITCH];
  const int k0 = blockIdx.x * TK, n0 = blockIdx.y * TN;
  const size_t mat_words = size_t(K) * N / 8;
  src += size_t(blockIdx.z) * mat_words;
  dst += size_t(blockIdx.z) * (mat_words / 4);
  const int row_words = N / 8;
  for (int i = threadIdx.x; i < TK * 32; i += 256) {
    const int row = i >> 5, wcol = i & 31;
    const int nw = n0 / 8 + wcol;
    tile[row * PITCH + wcol] = nw < row_words ? __ldcs(src + size_t(k0 + row) * row_words + nw) : 0u;
  }
  __syncthreads();
  const size_t units_per_group = size_t(K) / 8;
  for (int u = threadIdx.x; u < (TN / 4) * (TK / 8); u += 256) {
    const int c = u & (TK / 8 - 1), rg = u / (TK / 8);
    if (n0 + 4 * rg >= N) continue;
    const uint32_t *col = tile + (8 * c) * PITCH + (rg >> 1);
    uint32_t r[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) r[e] = col[e * PITCH];
    // the row group's four n sit in the low or the high half of each word
    const uint32_t pick = (rg & 1) ? 0x7632u : 0x5410u;
    const uint32_t X = __byte_perm(r[0], r[2], pick), Y = __byte_perm(r[4], r[6], pick);  // k = 0,2 | 4,6 (even k: nibbles 0..3)
    const uint32_t Z = __byte_perm(r[1], r[3], pick), W = __byte_perm(r[5], r[7], pick);  // k = 1,3 | 5,7 (odd k: nibbles 4..7)
    const uint32_t e01 = __byte_perm(X, Y, 0x6420), o01 = __byte_perm(Z, W, 0x6420);      // rows n, n+1 of k = 0,2,4,6 / 1,3,5,7
    const uint32_t e23 = __byte_perm(X, Y, 0x7531), o23 = __byte_perm(Z, W, 0x7531);      // rows n+2, n+3
    constexpr uint32_t LO = 0x0f0f0f0fu, BIAS = 0x88888888u;
    uint4 out;
    out.x = (squeeze_low_nibbles(e01 & LO) | (squeeze_low_nibbles(o01 & LO) << 16)) ^ BIAS;
    out.y = (squeeze_low_nibbles((e01 >> 4) & LO) | (squeeze_low_nibbles((o01 >> 4) & LO) << 16)) ^ BIAS;
    out.z = (squeeze_low_nibbles(e23 & LO) | (squeeze_low_nibbles(o23 & LO) << 16)) ^ BIAS;
    out.w = (squeeze_low_nibbles((e23 >> 4) & LO) | (squeeze_low_nibbles((o23 >> 4) & LO) << 16)) ^ BIAS;
    __stcs(dst + size_t(n0 / 4 + rg) * units_per_group + size_t(k0 / 8 + c), out);
  }
}

__global__ void pack_int4_kernel(uint8_t *__restrict__ dst, const int8_t *__restrict__ src, size_t n_packed) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n_packed;
       i += size_t(gridDim.x) * blockDim.x) {
    const char2 v = reinterpret_cast<const char2 *>(src)[i];
    dst[i] = uint8_t((uint8_t(v.x) & 0x0F) | (uint8_t(v.y) << 4));
  }
}

__global__ void unpack_int4_kernel(int8_t *__restrict__ dst, const uint8_t *__restrict__ src, size_t n_packed) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n_packed;
       i += size_t(gridDim.x) * blockDim.x) {
    const uint8_t b = src[i];
    char2 v;
    v.x = int8_t(int8_t(b << 4) >> 4);  // arithmetic shift sign-extends the low nibble
    v.y = int8_t(int8_t(b) >> 4);
    reinterpret_cast<char2 *>(dst)[i] = v;
  }
}

__global__ void preprocess_zeros_kernel(__half *__restrict__ dst, const __half *__restrict__ scales,
                                        const int8_t *__restrict__ zeros, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x) {
    // half(-z) is exact; one round-to-nearest multiply, as the host code does.
    dst[i] = __hmul(__int2half_rn(-int(zeros[i])), scales[i]);
  }
}

int grid_for(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  return int(g < 1 ? 1 : (g > 148 * 32 ? 148 * 32 : g));
}

}  // namespace
}  // namespace mgv

using namespace mgv;

extern "C" mgv_status mgv_pack_int4(void *dst, const void *src, size_t n_unpacked, mgv_stream_t s) {
  if (n_unpacked % 2) return fail(MGV_STATUS_INVALID_ARGUMENT, "pack_int4: odd element count %zu", n_unpacked);
  if (n_unpacked == 0) return MGV_STATUS_OK;
  if (!dst || !src) return fail(MGV_STATUS_INVALID_ARGUMENT, "pack_int4: null pointer");
  if (reinterpret_cast<uintptr_t>(src) % 2) return fail(MGV_STATUS_MISALIGNED, "pack_int4: src must be 2-byte aligned");
  const size_t np = n_unpacked / 2;
  pack_int4_kernel<<<grid_for(np, 256), 256, 0, s>>>(static_cast<uint8_t *>(dst), static_cast<const int8_t *>(src), np);
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_unpack_int4(void *dst, const void *src, size_t n_packed, mgv_stream_t s) {
  if (n_packed == 0) return MGV_STATUS_OK;
  if (!dst || !src) return fail(MGV_STATUS_INVALID_ARGUMENT, "unpack_int4: null pointer");
  if (reinterpret_cast<uintptr_t>(dst) % 2) return fail(MGV_STATUS_MISALIGNED, "unpack_int4: dst must be 2-byte aligned");
  unpack_int4_kernel<<<grid_for(n_packed, 256), 256, 0, s>>>(static_cast<int8_t *>(dst), static_cast<const uint8_t *>(src), n_packed);
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_preprocess_zeros(void *dst, const void *scales, const void *zeros, size_t n, mgv_stream_t s) {
  if (n == 0) return MGV_STATUS_OK;
  if (!dst || !scales || !zeros) return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_zeros: null pointer");
  preprocess_zeros_kernel<<<grid_for(n, 256), 256, 0, s>>>(static_cast<__half *>(dst), static_cast<const __half *>(scales),
                                                           static_cast<const int8_t *>(zeros), n);
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_preprocess_weights(void *dst, const void *src, const size_t *shape, int rank, int layout,
                                             int quant_type, mgv_stream_t s) {
  if (!shape || (rank != 2 && rank != 3))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: shape must be {K,N} or {E,K,N} (rank %d)", rank);
  if (quant_type == MGV_W4_AFP8)
    return fail(MGV_STATUS_UNSUPPORTED, "preprocess_weights: W4_AFP8 has no interleave rule and no kernel");
  if (quant_type != MGV_W4_A16 && quant_type != MGV_W8_A16)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: unknown quant_type %d", quant_type);
  if (layout != MGV_LAYOUT_ROW_MAJOR && layout != MGV_LAYOUT_COLUMN_MAJOR)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: unknown layout %d", layout);
  const int bits = quant_type == MGV_W4_A16 ? 4 : 8;
  const size_t E = rank == 3 ? shape[0] : 1, K = shape[rank - 2], N = shape[rank - 1];
  if (E == 0 || K == 0 || N == 0) return MGV_STATUS_OK;
  if (N % size_t(16 / bits))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: N=%zu must be a multiple of %d", N, 16 / bits);
  if (K % 8) return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: K=%zu must be a multiple of 8", K);
  if (layout == MGV_LAYOUT_ROW_MAJOR && ((N * bits / 8) % 32 || (K * bits / 8) % 32))
    return fail(MGV_STATUS_INVALID_ARGUMENT,
                "preprocess_weights: row-major input needs N*bits/8 and K*bits/8 multiples of 32 (N=%zu K=%zu)", N, K);
  if (K > 0x7fffffffu || N > 0x7fffffffu || E > 65535u)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: dimension too large");
  if (!dst || !src) return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: null pointer");
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) % 4)
    return fail(MGV_STATUS_MISALIGNED, "preprocess_weights: buffers must be 4-byte aligned");
  if (dst == src) return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: dst and src must not overlap");
  const bool rm_in = layout == MGV_LAYOUT_ROW_MAJOR;
  const size_t piece_k = bits == 4 ? 32 : 16;
  if (!rm_in && K % piece_k == 0 && (reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) % 16 == 0) {
    // no transpose: the direct kernel (experts are just more row groups: N is a multiple of the group height)
    const size_t groups = E * N / size_t(16 / bits), pieces = K / piece_k;
    const int blocks = int(std::min<size_t>((groups * pieces + 255) / 256, size_t(148) * 16));
    if (bits == 4)
      preprocess_direct_kernel<4><<<blocks, 256, 0, s>>>(static_cast<uint4 *>(dst), static_cast<const uint4 *>(src), K, groups, pieces);
    else
      preprocess_direct_kernel<8><<<blocks, 256, 0, s>>>(static_cast<uint4 *>(dst), static_cast<const uint4 *>(src), K, groups, pieces);
    MGV_CUDA_TRY(cudaGetLastError());
    return MGV_STATUS_OK;
  }
  if (rm_in && bits == 4 && K % 64 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 && (N + 255) / 256 <= 65535u) {
    dim3 grid(unsigned(K / 64), unsigned((N + 255) / 256), unsigned(E));
    preprocess_transpose4_kernel<<<grid, 256, 0, s>>>(static_cast<uint4 *>(dst), static_cast<const uint32_t *>(src), int(K), int(N));
    MGV_CUDA_TRY(cudaGetLastError());
    return MGV_STATUS_OK;
  }
  dim3 grid(unsigned((K + kTile - 1) / kTile), unsigned((N + kTile - 1) / kTile), unsigned(E));
  if (grid.y > 65535u) return fail(MGV_STATUS_INVALID_ARGUMENT, "preprocess_weights: N too large");
  auto *d = static_cast<uint32_t *>(dst);
  auto *p = static_cast<const uint32_t *>(src);
  const bool rm = layout == MGV_LAYOUT_ROW_MAJOR;
  if (bits == 4) {
    if (rm) preprocess_weights_kernel<4, true><<<grid, kThreads, 0, s>>>(d, p, int(K), int(N));
    else    preprocess_weights_kernel<4, false><<<grid, kThreads, 0, s>>>(d, p, int(K), int(N));
  } else {
    if (rm) preprocess_weights_kernel<8, true><<<grid, kThreads, 0, s>>>(d, p, int(K), int(N));
    else    preprocess_weights_kernel<8, false><<<grid, kThreads, 0, s>>>(d, p, int(K), int(N));
  }
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}
