// The fused dequantise + GEMV + reduce + epilogue kernel for sm_100a, and its launcher.
//
// It replaces the reference's device stack (gemv/kernel/mixed_gemv.h:133-254 and everything
// under gemv/threadblock, gemv/warp, gemv/thread, epilogue/threadblock) with one persistent,
// warp-specialised kernel:
//
//   * Work is cut into UNITS: one row tile (8 row groups = 32 rows for 4-bit, 16 rows for 8-bit
//     weights) times one K slice of 512.  Units are numbered tile-major and split evenly over
//     one thread block per SM, so every SM streams the same number of bytes whatever N and K
//     are (the reference launches ceil(N/64) blocks, fewer than there are SMs for N = 4096).
//   * A producer warp fills a ring of shared-memory stages, one unit per stage: the eight
//     contiguous 1 KB weight segments and the x slice with cp.async.bulk (TMA, no tensor map,
//     no multicast), the tile's scales/zeros with 4/8-byte cp.async; all complete on one
//     mbarrier per stage.  Eight consumer warps read 16-byte units from the ring.
//   * In the preprocessed layout one 16-byte unit holds 4 (or 2) output rows x 8 consecutive k.
//     Lane (g = lane/4, t = lane%4) of a consumer warp takes row group g and k chunk t of each
//     32-wide step, converts with the LOP3/PRMT magic-number sequence, applies scale (and zero)
//     in fp16 with separate roundings exactly as the reference does, and multiplies by x:
//       - SIMT family: fp32 FMAs on CUDA cores (fma.rn.f32.f16, sm_100+), 4 accumulators per
//         lane and batch row, shuffle reduction over the 4 k lanes at the end of a tile;
//       - MMA family: the lane's registers ARE the A fragment of mma.m16n8k16 (rows g and g+8,
//         a k permutation shared with the x fragment), fp32 accumulate, batch rows on the
//         8 (or 16) B columns; the k lanes are summed by the instruction.
//   * Warps split the steps of a stage, so a tile ends with a cross-warp sum through shared
//     memory.  A tile whose units are spread over several blocks is combined through a scratch
//     slot per block: the last block to arrive (a per-tile counter) adds the slots in block
//     order, which keeps the result deterministic, and runs the epilogue.
//   * Epilogue: out = half(alpha*acc + beta*bias), or the fp32 partial for K-split sharding.
//
// Every wait on an mbarrier is bounded (about a second); a wait that gives up records a code
// in the device error word, and the block keeps its barrier protocol intact while skipping work,
// so the launch always terminates.
#include <algorithm>
#include <cstring>
#include <mutex>

#include "mgv_common.cuh"

namespace mgv {

constexpr int KS = 512;                       // K elements per unit / stage
constexpr int RG = 8;                         // row groups per tile
constexpr int SEG_BYTES = KS / 8 * 16;        // one row group's bytes in a stage
constexpr int SEG_PITCH = SEG_BYTES + 64;     // +64: quarter-warp 16-byte reads hit 32 distinct banks
constexpr int X_PITCH = KS * 2 + 64;
constexpr int MAX_GPS = KS / 64;              // scale groups per stage, at most
constexpr int NW = 8;                         // consumer warps
constexpr int THREADS = (NW + 1) * 32;
constexpr int VAR_SIMT = 1, VAR_MMA = 2;
constexpr int kSlotFloats = 16 * 32;  // largest batch bucket x largest tile: one scratch slot size for all kernels

struct GemvParams {
  const uint8_t *w;
  const __half *x;
  const __half *scale;
  const __half *zero;
  const __half *bias;
  void *out;
  float *ws_slots;   // [grid][2][TILE_ROWS*MB] partial sums of split tiles
  int *ws_counters;  // [batch*tiles] arrivals per split tile (zero between launches)
  int *err;
  int64_t ldx, ldd;
  int64_t bs_w, bs_x, bs_scale, bs_bias, bs_out;
  float alpha, beta;
  int M, N, K;
  int group_size;
  int gshift;        // log2(group_size) when several groups fit a stage, else -1 (one group per stage)
  int tiles;         // row tiles per problem
  int upt;           // units per tile = ceil(K / KS)
  int total_tiles;   // batch_count * tiles
  int align_tiles;   // 1: blocks own whole tiles (no scratch); 0: blocks own equal unit ranges
  int stages;
  int flags;
};

template <int BITS, int MB>
struct Geometry {
  static constexpr int RPG = 16 / BITS;            // rows per 16-byte unit
  static constexpr int TILE_ROWS = RG * RPG;
  static constexpr int S_BYTES = MAX_GPS * TILE_ROWS * 2;
  static constexpr int W_OFF = 0;
  static constexpr int X_OFF = RG * SEG_PITCH;
  static constexpr int S_OFF = X_OFF + MB * X_PITCH;
  static constexpr int Z_OFF = S_OFF + S_BYTES;
  static constexpr int STAGE_BYTES = ((Z_OFF + S_BYTES) + 127) / 128 * 128;
  static constexpr int RED_FLOATS = NW * MB * TILE_ROWS;
  // barriers (2 per stage, up to 32 stages) + flags, then the reduction buffer, then the ring
  static constexpr int HEAD_BYTES = 1024;
  static constexpr int RED_OFF = HEAD_BYTES;
  static constexpr int RING_OFF = (RED_OFF + RED_FLOATS * 4 + 127) / 128 * 128;
};

__device__ __forceinline__ uint32_t dup_lo(uint32_t v) { return __byte_perm(v, v, 0x1010); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t v) { return __byte_perm(v, v, 0x3232); }

__device__ __forceinline__ uint32_t hmul2_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hadd2_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// c_lo += a.lo*b.lo ; c_hi += a.hi*b.hi with fp16 inputs and fp32 accumulate (exact product,
// one rounding), the arithmetic of gemv/thread/mma.h:83-96.
__device__ __forceinline__ void fma_mixed(uint32_t a2, uint32_t b2, float &c_lo, float &c_hi) {
  asm("{\n\t.reg .f16 al, ah, bl, bh;\n\t"
      "mov.b32 {al, ah}, %2;\n\t"
      "mov.b32 {bl, bh}, %3;\n\t"
      "fma.rn.f32.f16 %0, al, bl, %0;\n\t"
      "fma.rn.f32.f16 %1, ah, bh, %1;\n\t}"
      : "+f"(c_lo), "+f"(c_hi)
      : "r"(a2), "r"(b2));
}

__device__ __forceinline__ float apply_act(float v, int flags) {
  if (flags & MGV_FLAG_ACT_RELU) v = fmaxf(v, 0.0f);
  if (flags & MGV_FLAG_ACT_SILU) v = v / (1.0f + __expf(-v));
  return v;
}

// Block that owns unit u when U units are dealt to G blocks as [c*U/G, (c+1)*U/G).
__device__ __forceinline__ int owner_of_unit(long long u, long long U, int G) {
  return int(((u + 1) * G - 1) / U);
}

template <int BITS, bool HAS_ZERO, int VAR, int MB>
__global__ void __launch_bounds__(THREADS, 1) gemv_kernel(const GemvParams p) {
  using Geo = Geometry<BITS, MB>;
  constexpr int RPG = Geo::RPG;
  constexpr int TILE_ROWS = Geo::TILE_ROWS;
  constexpr int NACC = VAR == VAR_MMA ? (MB / 8) * (RPG / 2) * 4 : MB * RPG * 2;
  static_assert(VAR == VAR_SIMT || MB % 8 == 0, "MMA family covers 8 or 16 batch columns");

  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty_bar = full_bar + 32;
  volatile int *sh_abort = reinterpret_cast<volatile int *>(smem + 512);
  volatile int *sh_last = reinterpret_cast<volatile int *>(smem + 516);
  float *red = reinterpret_cast<float *>(smem + Geo::RED_OFF);
  uint8_t *ring = smem + Geo::RING_OFF;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int NS = p.stages;
  const int G = gridDim.x, cta = blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full_bar[s], 33);  // producer lane 0 (with the byte count) + 32 cp.async arrivals
      mbar_init(&empty_bar[s], NW);
    }
    *sh_abort = 0;
    *sh_last = 0;
    mbar_fence_init();
  }
  __syncthreads();

  const long long U = (long long)p.total_tiles * p.upt;
  long long u_begin, u_end;
  if (p.align_tiles) {
    u_begin = ((long long)cta * p.total_tiles / G) * p.upt;
    u_end = ((long long)(cta + 1) * p.total_tiles / G) * p.upt;
  } else {
    u_begin = (long long)cta * U / G;
    u_end = (long long)(cta + 1) * U / G;
  }

  if (warp == NW) {
    // ======================= producer warp =======================
    bool skip = false;
    for (long long u = u_begin; u < u_end; ++u) {
      const int it = int(u - u_begin), s = it % NS;
      if (*sh_abort) skip = true;
      if (!skip && it >= NS) {
        if (!mbar_wait_bounded(&empty_bar[s], ((it / NS) - 1) & 1)) {
          atomicOr(p.err, DEVERR_EMPTY_WAIT);
          *sh_abort = 1;
          skip = true;
        }
      }
      skip = __any_sync(0xffffffffu, skip);
      if (skip) continue;
      const int tg = int(u / p.upt), ks = int(u % p.upt);
      const int b = tg / p.tiles, tile = tg % p.tiles;
      const int k0 = ks * KS, kn = min(KS, p.K - k0);
      const int n0 = tile * TILE_ROWS;
      const int rgv = min(RG, (p.N - n0) / RPG);
      uint8_t *st = ring + size_t(s) * Geo::STAGE_BYTES;
      if (lane == 0) {
        const uint32_t seg = uint32_t(kn / 8 * 16);
        mbar_arrive_expect_tx(&full_bar[s], uint32_t(rgv) * seg + uint32_t(p.M) * uint32_t(kn * 2));
        const uint8_t *wb = p.w + size_t(b) * p.bs_w + (size_t(n0 / RPG) * (p.K / 8) + k0 / 8) * 16;
        for (int r = 0; r < rgv; ++r)
          bulk_g2s(st + Geo::W_OFF + r * SEG_PITCH, wb + size_t(r) * (p.K / 8) * 16, seg, &full_bar[s]);
        const __half *xb = p.x + size_t(b) * p.bs_x + k0;
        for (int m = 0; m < p.M; ++m)
          bulk_g2s(st + Geo::X_OFF + m * X_PITCH, xb + size_t(m) * p.ldx, uint32_t(kn * 2), &full_bar[s]);
      }
      {
        const int g_first = p.gshift >= 0 ? (k0 >> p.gshift) : (k0 / p.group_size);
        const int ng = p.gshift >= 0 ? (kn >> p.gshift) : 1;
        const __half *sb = p.scale + size_t(b) * p.bs_scale + size_t(g_first) * p.N + n0;
        const __half *zb = HAS_ZERO ? p.zero + size_t(b) * p.bs_scale + size_t(g_first) * p.N + n0 : nullptr;
        for (int i = lane; i < ng * RG; i += 32) {
          const int gl = i / RG, r = i % RG;
          if (r < rgv) {
            const int dst = (gl * TILE_ROWS + r * RPG) * 2;
            cp_async_small<RPG * 2>(st + Geo::S_OFF + dst, sb + size_t(gl) * p.N + r * RPG);
            if (HAS_ZERO) cp_async_small<RPG * 2>(st + Geo::Z_OFF + dst, zb + size_t(gl) * p.N + r * RPG);
          }
        }
        cp_async_arrive_noinc(&full_bar[s]);
      }
    }
    if (*sh_abort) {
      // Unwinding after a timeout: do not leave the block while copies may still land in its
      // shared memory.  Wait (bounded) for the phase of every stage this warp filled last.
      const int n_it = int(u_end - u_begin);
      for (int it = max(0, n_it - NS); it < n_it; ++it)
        if (!mbar_wait_bounded(&full_bar[it % NS], (it / NS) & 1)) atomicOr(p.err, DEVERR_DRAIN_WAIT);
    }
    return;
  }

  // ======================= consumer warps =======================
  const int g = lane >> 2, t = lane & 3;
  const int ctid = threadIdx.x;  // 0 .. NW*32-1
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
  bool skip = false;

  for (long long u = u_begin; u < u_end; ++u) {
    const int it = int(u - u_begin), s = it % NS;
    const int tg = int(u / p.upt), ks = int(u % p.upt);
    const int k0 = ks * KS, kn = min(KS, p.K - k0);
    uint8_t *st = ring + size_t(s) * Geo::STAGE_BYTES;

    if (*sh_abort) skip = true;
    if (!skip && !mbar_wait_bounded(&full_bar[s], (it / NS) & 1)) {
      atomicOr(p.err, DEVERR_FULL_WAIT);
      *sh_abort = 1;
      skip = true;
    }
    skip = __any_sync(0xffffffffu, skip);

    if (!skip) {
      const int steps = kn / 32;
      for (int sp = warp; sp < steps; sp += NW) {
        const int coff = (4 * sp + t) * 16;
        const uint4 wv = lds128(st + Geo::W_OFF + g * SEG_PITCH + coff);
        const int gl = p.gshift >= 0 ? ((32 * sp) >> p.gshift) : 0;
        const int soff = (gl * TILE_ROWS + g * RPG) * 2;
        // ---- dequantise the 16-byte unit: hh[row][pair] = half2 of (k, k+1) ----
        uint32_t hh[RPG][4];
        if constexpr (BITS == 4) {
          const uint2 sv = *reinterpret_cast<const uint2 *>(st + Geo::S_OFF + soff);
          const uint32_t s2[4] = {dup_lo(sv.x), dup_hi(sv.x), dup_lo(sv.y), dup_hi(sv.y)};
          uint32_t z2[4] = {0, 0, 0, 0};
          if (HAS_ZERO) {
            const uint2 zv = *reinterpret_cast<const uint2 *>(st + Geo::Z_OFF + soff);
            z2[0] = dup_lo(zv.x); z2[1] = dup_hi(zv.x); z2[2] = dup_lo(zv.y); z2[3] = dup_hi(zv.y);
          }
          const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            cvt_u4x8(wr[j], hh[j]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              hh[j][i] = hmul2_rn(hh[j][i], s2[j]);
              if (HAS_ZERO) hh[j][i] = hadd2_rn(hh[j][i], z2[j]);
            }
          }
        } else {
          const uint32_t sv = *reinterpret_cast<const uint32_t *>(st + Geo::S_OFF + soff);
          const uint32_t s2[2] = {dup_lo(sv), dup_hi(sv)};
          uint32_t z2[2] = {0, 0};
          if (HAS_ZERO) {
            const uint32_t zv = *reinterpret_cast<const uint32_t *>(st + Geo::Z_OFF + soff);
            z2[0] = dup_lo(zv); z2[1] = dup_hi(zv);
          }
          const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint32_t lo[2], hi[2];
            cvt_u8x4(wr[2 * j], lo);
            cvt_u8x4(wr[2 * j + 1], hi);
            hh[j][0] = lo[0]; hh[j][1] = lo[1]; hh[j][2] = hi[0]; hh[j][3] = hi[1];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              hh[j][i] = hmul2_rn(hh[j][i], s2[j]);
              if (HAS_ZERO) hh[j][i] = hadd2_rn(hh[j][i], z2[j]);
            }
          }
        }
        // ---- multiply-accumulate ----
        if constexpr (VAR == VAR_MMA) {
#pragma unroll
          for (int c8 = 0; c8 < MB / 8; ++c8) {
            const int xr = c8 * 8 + g;  // this lane supplies batch column xr of the B fragment
            uint4 xv = make_uint4(0, 0, 0, 0);
            if (xr < p.M) xv = lds128(st + Geo::X_OFF + xr * X_PITCH + coff);
#pragma unroll
            for (int q = 0; q < RPG / 2; ++q) {
              float(&c)[4] = *reinterpret_cast<float(*)[4]>(&acc[(c8 * (RPG / 2) + q) * 4]);
              mma_16816(c, hh[2 * q][0], hh[2 * q + 1][0], hh[2 * q][1], hh[2 * q + 1][1], xv.x, xv.y);
              mma_16816(c, hh[2 * q][2], hh[2 * q + 1][2], hh[2 * q][3], hh[2 * q + 1][3], xv.z, xv.w);
            }
          }
        } else {
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            if (m < p.M) {
              const uint4 xv = lds128(st + Geo::X_OFF + m * X_PITCH + coff);
#pragma unroll
              for (int j = 0; j < RPG; ++j) {
                float &lo = acc[(m * RPG + j) * 2], &hi = acc[(m * RPG + j) * 2 + 1];
                fma_mixed(hh[j][0], xv.x, lo, hi);
                fma_mixed(hh[j][1], xv.y, lo, hi);
                fma_mixed(hh[j][2], xv.z, lo, hi);
                fma_mixed(hh[j][3], xv.w, lo, hi);
              }
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);

    // ---- end of this block's share of the tile? ----
    const bool last_of_tile = ks == p.upt - 1;
    if (!last_of_tile && u != u_end - 1) continue;

    // cross-warp sum through shared memory: red[warp][m][row]
    if constexpr (VAR == VAR_MMA) {
#pragma unroll
      for (int c8 = 0; c8 < MB / 8; ++c8)
#pragma unroll
        for (int q = 0; q < RPG / 2; ++q)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = c8 * 8 + 2 * t + (e & 1);
            const int row = g * RPG + 2 * q + (e >> 1);
            if (col < p.M) red[(warp * MB + col) * TILE_ROWS + row] = acc[(c8 * (RPG / 2) + q) * 4 + e];
          }
    } else {
#pragma unroll
      for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int j = 0; j < RPG; ++j) {
          float v = acc[(m * RPG + j) * 2] + acc[(m * RPG + j) * 2 + 1];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if (t == 0 && m < p.M) red[(warp * MB + m) * TILE_ROWS + g * RPG + j] = v;
        }
    }
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
    named_bar_sync(1, NW * 32);

    const int b = tg / p.tiles, tile = tg % p.tiles;
    const int n0 = tile * TILE_ROWS;
    const long long tile_u0 = (long long)tg * p.upt;
    const bool whole = last_of_tile && (u_begin <= tile_u0);  // this block saw every unit of the tile
    const int n_out = p.M * TILE_ROWS;

    auto epilogue = [&](int i, float v) {
      const int m = i / TILE_ROWS, n = n0 + i % TILE_ROWS;
      if (n >= p.N) return;
      const size_t o = size_t(b) * p.bs_out + size_t(m) * p.ldd + n;
      if (p.flags & MGV_FLAG_OUT_F32_PARTIAL) {
        static_cast<float *>(p.out)[o] = p.alpha * v;
      } else {
        float r = p.alpha * v;
        if (p.bias) r += p.beta * __half2float(p.bias[size_t(b) * p.bs_bias + n]);
        static_cast<__half *>(p.out)[o] = __float2half_rn(apply_act(r, p.flags));
      }
    };

    if (whole) {
      for (int i = ctid; i < n_out; i += NW * 32) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[w * MB * TILE_ROWS + i];
        epilogue(i, v);
      }
    } else {
      // Split tile: park this block's sum in its scratch slot, count the arrival, and let the
      // last block add all slots in block order.
      const int first_c = owner_of_unit(tile_u0, U, G);
      const int last_c = owner_of_unit(tile_u0 + p.upt - 1, U, G);
      const int which = (u_begin / p.upt == tg) ? 0 : 1;  // 0: the tile this block's range starts in
      float *slot = p.ws_slots + (size_t(cta) * 2 + which) * kSlotFloats;
      for (int i = ctid; i < n_out; i += NW * 32) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[w * MB * TILE_ROWS + i];
        __stcg(slot + i, v);
      }
      __threadfence();
      named_bar_sync(1, NW * 32);
      if (ctid == 0) {
        const int prev = atomicAdd(p.ws_counters + tg, 1);
        const int last = prev == (last_c - first_c);
        if (last) p.ws_counters[tg] = 0;  // leave the scratch ready for the next launch
        *sh_last = last;
      }
      named_bar_sync(1, NW * 32);
      if (*sh_last) {
        __threadfence();
        for (int i = ctid; i < n_out; i += NW * 32) {
          float v = 0.0f;
          for (int c = first_c; c <= last_c; ++c) {
            // block c's slot for this tile: 0 if the tile is where its range starts, else 1
            const long long cb = (long long)c * U / G;
            const int wc = (cb / p.upt == tg) ? 0 : 1;
            v += __ldcg(p.ws_slots + (size_t(c) * 2 + wc) * kSlotFloats + i);
          }
          epilogue(i, v);
        }
      }
    }
    named_bar_sync(1, NW * 32);  // red and sh_last are reused by the next tile
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

struct DeviceInfo {
  int sms = 0;
  int smem_optin = 0;
  int *err_word = nullptr;
};

__device__ int g_device_error_word;

static DeviceInfo *device_info(mgv_status *st) {
  static DeviceInfo infos[64];
  static bool ready[64];
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *st = cuda_fail(e, "cudaGetDevice");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ready[dev]) {
    DeviceInfo d;
    if ((e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess ||
        (e = cudaGetSymbolAddress(reinterpret_cast<void **>(&d.err_word), g_device_error_word)) != cudaSuccess) {
      *st = cuda_fail(e, "device query");
      return nullptr;
    }
    infos[dev] = d;
    ready[dev] = true;
  }
  return &infos[dev];
}

int *device_error_word() {
  mgv_status st = MGV_STATUS_OK;
  DeviceInfo *d = device_info(&st);
  return d ? d->err_word : nullptr;
}

namespace {

struct Plan {
  int variant, mb, bits, has_zero;
  int tile_rows, tiles, upt, total_tiles;
  int grid, stages, smem, stage_bytes, ring_off;
  int align_tiles, split_tiles, gshift, group;
  size_t ws_counter_bytes, ws_bytes;
};

template <int BITS, int MB>
void geometry(Plan &pl) {
  using Geo = Geometry<BITS, MB>;
  pl.tile_rows = Geo::TILE_ROWS;
  pl.stage_bytes = Geo::STAGE_BYTES;
  pl.ring_off = Geo::RING_OFF;
}

int count_split_tiles(long long U, int upt, int G) {
  // tiles whose units are owned by more than one block under the equal-unit split
  int n = 0;
  long long prev_tile = -1;
  for (int c = 1; c < G; ++c) {
    const long long ub = (long long)c * U / G;
    if (ub % upt != 0 && ub / upt != prev_tile) {  // a block boundary strictly inside a tile
      ++n;
      prev_tile = ub / upt;
    }
  }
  return n;
}

mgv_status make_plan(const mgv_gemv_args &a, const DeviceInfo &dev, bool have_ws_hint, Plan &pl) {
  if (a.struct_size != int32_t(sizeof(mgv_gemv_args)))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: struct_size %d != %zu (header/library mismatch)", a.struct_size,
                sizeof(mgv_gemv_args));
  if (a.weight_bits != 4 && a.weight_bits != 8)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: weight_bits must be 4 or 8, got %d", a.weight_bits);
  if (a.M < 1 || a.M > 16) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: M must be 1..16, got %d", a.M);
  if (a.N < 1 || a.K < 1) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: N and K must be positive (N=%d K=%d)", a.N, a.K);
  const int rpg = 16 / a.weight_bits;
  if (a.N % rpg) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: N=%d must be a multiple of %d", a.N, rpg);
  if (a.K % 64) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: K=%d must be a multiple of 64", a.K);
  if (a.quant_op != MGV_QUANT_PER_COLUMN_SCALE_ONLY && a.quant_op != MGV_QUANT_FINEGRAINED_SCALE_ONLY &&
      a.quant_op != MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: quant_op %d is not a WeightOnlyQuantOp mode", a.quant_op);
  int group = a.quant_op == MGV_QUANT_PER_COLUMN_SCALE_ONLY ? a.K : a.group_size;
  if (group < 64) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: group_size %d is below 64", group);
  if (a.K % group) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: K=%d is not a multiple of group_size %d", a.K, group);
  const bool pow2 = (group & (group - 1)) == 0;
  if (!pow2 && group != a.K)
    return fail(MGV_STATUS_UNSUPPORTED, "gemv: group_size %d must be a power of two or equal K", group);
  pl.group = group;
  pl.gshift = (pow2 && group <= KS) ? __builtin_ctz(group) : -1;
  pl.has_zero = a.quant_op == MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS;
  if (!a.weights || !a.x || !a.scale || !a.out) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: null weights/x/scale/out");
  if (pl.has_zero && !a.zero) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: FINEGRAINED_SCALE_AND_ZEROS needs zero");
  if (a.flags & ~(MGV_FLAG_OUT_F32_PARTIAL | MGV_FLAG_ACT_RELU | MGV_FLAG_ACT_SILU))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: unknown flag bits 0x%x", a.flags);
  if ((a.flags & MGV_FLAG_ACT_RELU) && (a.flags & MGV_FLAG_ACT_SILU))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: choose one activation");
  if (a.ldx < a.K || a.ldd < a.N) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: ldx < K or ldd < N");
  const int batch = a.batch_count <= 0 ? 1 : a.batch_count;
  auto mis = [](const void *p, size_t al) { return reinterpret_cast<uintptr_t>(p) % al != 0; };
  if (mis(a.weights, 16) || mis(a.x, 16)) return fail(MGV_STATUS_MISALIGNED, "gemv: weights and x must be 16-byte aligned");
  if (a.ldx % 8) return fail(MGV_STATUS_MISALIGNED, "gemv: ldx=%lld must be a multiple of 8", (long long)a.ldx);
  if (mis(a.scale, rpg * 2) || (pl.has_zero && mis(a.zero, rpg * 2)))
    return fail(MGV_STATUS_MISALIGNED, "gemv: scale/zero must be %d-byte aligned", rpg * 2);
  if (mis(a.out, (a.flags & MGV_FLAG_OUT_F32_PARTIAL) ? 4 : 2) || (a.bias && mis(a.bias, 2)))
    return fail(MGV_STATUS_MISALIGNED, "gemv: out/bias misaligned");
  if (batch > 1 && (a.batch_stride_weights % 16 || a.batch_stride_x % 8 || a.batch_stride_scale % rpg))
    return fail(MGV_STATUS_MISALIGNED, "gemv: batch strides break the 16-byte / 8-element rules");

  // ---- kernel family and batch bucket ----
  int variant = a.variant;
  if (variant == MGV_VARIANT_AUTO) variant = MGV_VARIANT_MMA;
  if (variant != MGV_VARIANT_SIMT && variant != MGV_VARIANT_MMA)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: unknown variant %d", a.variant);
  if (variant == MGV_VARIANT_SIMT && a.M > 4)
    return fail(MGV_STATUS_UNSUPPORTED, "gemv: the SIMT family covers M <= 4 (M=%d)", a.M);
  pl.variant = variant;
  pl.bits = a.weight_bits;
  pl.mb = variant == MGV_VARIANT_SIMT ? (a.M == 1 ? 1 : (a.M == 2 ? 2 : 4)) : (a.M <= 8 ? 8 : 16);
#define MGV_GEO(B, MBV) if (pl.bits == B && pl.mb == MBV) geometry<B, MBV>(pl);
  MGV_GEO(4, 1) MGV_GEO(4, 2) MGV_GEO(4, 4) MGV_GEO(4, 8) MGV_GEO(4, 16)
  MGV_GEO(8, 1) MGV_GEO(8, 2) MGV_GEO(8, 4) MGV_GEO(8, 8) MGV_GEO(8, 16)
#undef MGV_GEO
  pl.tiles = (a.N + pl.tile_rows - 1) / pl.tile_rows;
  pl.upt = (a.K + KS - 1) / KS;
  const long long total_tiles = (long long)pl.tiles * batch;
  if (total_tiles > 0x3fffffff) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: too many row tiles");
  pl.total_tiles = int(total_tiles);
  const long long U = total_tiles * pl.upt;
  pl.grid = int(std::min<long long>(dev.sms, U));
  const int max_stages = std::min(32, (dev.smem_optin - pl.ring_off) / pl.stage_bytes);
  if (max_stages < 2) return fail(MGV_STATUS_UNSUPPORTED, "gemv: not enough shared memory for two stages");
  const long long per_block = (U + pl.grid - 1) / pl.grid;
  pl.stages = int(std::max<long long>(2, std::min<long long>(max_stages, per_block)));
  pl.smem = pl.ring_off + pl.stages * pl.stage_bytes;
  pl.ws_counter_bytes = (size_t(pl.total_tiles) * 4 + 255) / 256 * 256;
  pl.ws_bytes = pl.ws_counter_bytes + size_t(dev.sms) * 2 * kSlotFloats * 4;
  pl.split_tiles = count_split_tiles(U, pl.upt, pl.grid);
  // Without scratch, blocks own whole tiles; with it, equal unit ranges.
  pl.align_tiles = (pl.split_tiles == 0 || !have_ws_hint) ? 1 : 0;
  if (pl.align_tiles) {
    pl.grid = int(std::min<long long>(pl.grid, total_tiles));
    pl.split_tiles = 0;
  }
  return MGV_STATUS_OK;
}

template <int BITS, bool HZ, int VAR, int MB>
mgv_status launch(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  auto kern = gemv_kernel<BITS, HZ, VAR, MB>;
  static int configured_smem[64];
  int dev = 0;
  MGV_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_smem[dev % 64] < pl.smem) {
    // raise to the device maximum once; later launches with any stage count fit
    int optin = 0;
    MGV_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    MGV_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, optin));
    configured_smem[dev % 64] = optin;
  }
  kern<<<pl.grid, THREADS, pl.smem, s>>>(p);
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}

template <int BITS, bool HZ>
mgv_status dispatch_family(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.variant == MGV_VARIANT_SIMT) {
    if (pl.mb == 1) return launch<BITS, HZ, VAR_SIMT, 1>(p, pl, s);
    if (pl.mb == 2) return launch<BITS, HZ, VAR_SIMT, 2>(p, pl, s);
    return launch<BITS, HZ, VAR_SIMT, 4>(p, pl, s);
  }
  if (pl.mb == 8) return launch<BITS, HZ, VAR_MMA, 8>(p, pl, s);
  return launch<BITS, HZ, VAR_MMA, 16>(p, pl, s);
}

}  // namespace
}  // namespace mgv

using namespace mgv;

extern "C" void mgv_gemv_args_init(mgv_gemv_args *a) {
  if (!a) return;
  std::memset(a, 0, sizeof(*a));
  a->struct_size = int32_t(sizeof(*a));
  a->alpha = 1.0f;
  a->beta = 1.0f;
  a->batch_count = 1;
  a->variant = MGV_VARIANT_AUTO;
}

extern "C" mgv_status mgv_gemv_workspace_size(const mgv_gemv_args *a, size_t *bytes) {
  if (!a || !bytes) return fail(MGV_STATUS_INVALID_ARGUMENT, "workspace_size: null argument");
  mgv_status st = MGV_STATUS_OK;
  DeviceInfo *dev = device_info(&st);
  if (!dev) return st;
  Plan pl{};
  // pointer checks do not matter for sizing: size with placeholders where the caller has none yet
  mgv_gemv_args tmp = *a;
  alignas(16) static char placeholder[16];
  if (!tmp.weights) tmp.weights = placeholder;
  if (!tmp.x) tmp.x = placeholder;
  if (!tmp.scale) tmp.scale = placeholder;
  if (!tmp.zero) tmp.zero = placeholder;
  if (!tmp.out) tmp.out = placeholder;
  if (tmp.ldx == 0) tmp.ldx = tmp.K;
  if (tmp.ldd == 0) tmp.ldd = tmp.N;
  if ((st = make_plan(tmp, *dev, true, pl)) != MGV_STATUS_OK) return st;
  *bytes = pl.split_tiles ? pl.ws_bytes : 0;
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_workspace_init(void *ws, size_t bytes, mgv_stream_t s) {
  if (bytes == 0) return MGV_STATUS_OK;
  if (!ws) return fail(MGV_STATUS_INVALID_ARGUMENT, "workspace_init: null workspace");
  MGV_CUDA_TRY(cudaMemsetAsync(ws, 0, bytes, s));
  return MGV_STATUS_OK;
}

static mgv_status plan_for(const mgv_gemv_args *a, Plan &pl, DeviceInfo **dev_out) {
  if (!a) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: null args");
  mgv_status st = MGV_STATUS_OK;
  DeviceInfo *dev = device_info(&st);
  if (!dev) return st;
  *dev_out = dev;
  const bool have_ws = a->workspace != nullptr;
  if ((st = make_plan(*a, *dev, have_ws, pl)) != MGV_STATUS_OK) return st;
  if (!pl.align_tiles) {
    if (reinterpret_cast<uintptr_t>(a->workspace) % 256)
      return fail(MGV_STATUS_MISALIGNED, "gemv: workspace must be 256-byte aligned");
    if (a->workspace_bytes < pl.ws_bytes)
      return fail(MGV_STATUS_WORKSPACE_TOO_SMALL, "gemv: workspace has %zu bytes, the shape needs %zu", a->workspace_bytes,
                  pl.ws_bytes);
  }
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_gemv_launch_info(const mgv_gemv_args *a, mgv_launch_info *info) {
  if (!info) return fail(MGV_STATUS_INVALID_ARGUMENT, "launch_info: null info");
  Plan pl{};
  DeviceInfo *dev = nullptr;
  mgv_status st = plan_for(a, pl, &dev);
  if (st != MGV_STATUS_OK) return st;
  info->variant = pl.variant;
  info->grid = pl.grid;
  info->block = THREADS;
  info->stages = pl.stages;
  info->smem_bytes = pl.smem;
  info->tile_rows = pl.tile_rows;
  info->k_slice = KS;
  info->split_tiles = pl.split_tiles;
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_gemv(const mgv_gemv_args *a, mgv_stream_t s) {
  Plan pl{};
  DeviceInfo *dev = nullptr;
  mgv_status st = plan_for(a, pl, &dev);
  if (st != MGV_STATUS_OK) return st;
  GemvParams p{};
  p.w = static_cast<const uint8_t *>(a->weights);
  p.x = static_cast<const __half *>(a->x);
  p.scale = static_cast<const __half *>(a->scale);
  p.zero = pl.has_zero ? static_cast<const __half *>(a->zero) : nullptr;
  p.bias = (a->flags & MGV_FLAG_OUT_F32_PARTIAL) ? nullptr : static_cast<const __half *>(a->bias);
  p.out = a->out;
  p.ws_counters = static_cast<int *>(a->workspace);
  p.ws_slots = a->workspace ? reinterpret_cast<float *>(static_cast<uint8_t *>(a->workspace) + pl.ws_counter_bytes) : nullptr;
  p.err = dev->err_word;
  p.ldx = a->ldx; p.ldd = a->ldd;
  p.bs_w = a->batch_stride_weights; p.bs_x = a->batch_stride_x; p.bs_scale = a->batch_stride_scale;
  p.bs_bias = a->batch_stride_bias; p.bs_out = a->batch_stride_out;
  p.alpha = a->alpha; p.beta = a->beta;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.group_size = pl.group; p.gshift = pl.gshift;
  p.tiles = pl.tiles; p.upt = pl.upt; p.total_tiles = pl.total_tiles;
  p.align_tiles = pl.align_tiles; p.stages = pl.stages; p.flags = a->flags;
  if (pl.bits == 4) return pl.has_zero ? dispatch_family<4, true>(p, pl, s) : dispatch_family<4, false>(p, pl, s);
  return pl.has_zero ? dispatch_family<8, true>(p, pl, s) : dispatch_family<8, false>(p, pl, s);
}

extern "C" mgv_status mgv_device_error_state(int *state) {
  if (!state) return fail(MGV_STATUS_INVALID_ARGUMENT, "device_error_state: null state");
  MGV_CUDA_TRY(cudaDeviceSynchronize());
  int v = 0;
  MGV_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_device_error_word, sizeof(int)));
  if (v) {
    const int zero = 0;
    MGV_CUDA_TRY(cudaMemcpyToSymbol(g_device_error_word, &zero, sizeof(int)));
  }
  *state = v;
  return v ? fail(MGV_STATUS_DEVICE_TIMEOUT, "a bounded device wait gave up (code 0x%x)", v) : MGV_STATUS_OK;
}
