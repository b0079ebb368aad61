// The steady-state GEMV kernel with x staged in shared memory, and its launcher.
#include "mgv_gemv_parts.cuh"

namespace mgv {

// ------------------------------------------------------------------------------------------
// The steady-state kernel of the common decode case: MMA family, M <= 8, x staged in shared
// memory, K a multiple of 128 (at least 2048), N a multiple of the tile height, one problem,
// whole tiles per block, groups of 64 (TWO: two per item) or of 128 and more.  Same arithmetic
// as gemv_kernel for these shapes; what differs is the bookkeeping around an item, which
// dominated its instruction count: offsets instead of cursors, a compile-time ring depth, one
// predicate for all copies of an item, compile-time shared-memory offsets and, for 4-bit
// weights, accumulators that start from the item's correction term instead of adding it
// afterwards.
//
// Shared memory: [part: slots x 16 warps x M x tile rows floats][table][x][rings], offsets from
// the plan.  4-bit weights use the offset trick: table entry (32 bytes) of group h of item ki
// and lane quarter t, at (ki * groups per item + h) * 128 + t * 32, is {c0, c1, c0, c1, s0, s1, -, -}
// with c = -(1032*sum of x on the lo pairs + 72*sum on the hi pairs) and s = sum of x over the
// group's k for batch columns 2t and 2t+1.  Ring slot: [4 steps][32 lanes] 16 B weights, then
// [groups][32 lanes] SB bytes of scales, then the same of zeros.
// ------------------------------------------------------------------------------------------
// All copies of one 128-k item under one predicate, closed by the commit of the group (an item
// that is switched off still commits an empty group, which keeps the group count uniform).
// SB: bytes of scales per lane and group; the second group's scales sit 32*SB behind the first,
// the zeros behind the scales in the same order.
#define MGV_LEAN_W                                              \
  "@q cp.async.cg.shared.global [%0], [%1], 16;\n\t"            \
  "@q cp.async.cg.shared.global [%0+512], [%1+64], 16;\n\t"     \
  "@q cp.async.cg.shared.global [%0+1024], [%1+128], 16;\n\t"   \
  "@q cp.async.cg.shared.global [%0+1536], [%1+192], 16;\n\t"
template <int SB, bool HAS_ZERO, bool TWO>
__device__ __forceinline__ void lean_copy_item(uint32_t wd, const void *wp, uint32_t sd, const __half *sp, const __half *zp,
                                               uint32_t n_cols, bool on) {
  if constexpr (!HAS_ZERO && !TWO) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %4, 0;\n\t" MGV_LEAN_W
                 "@q cp.async.ca.shared.global [%2], [%3], %5;\n\t"
                 "cp.async.commit_group;\n\t}" ::"r"(wd), "l"(wp), "r"(sd), "l"(sp), "r"(int(on)), "n"(SB)
                 : "memory");
  } else if constexpr (HAS_ZERO && !TWO) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t" MGV_LEAN_W
                 "@q cp.async.ca.shared.global [%2], [%3], %6;\n\t"
                 "@q cp.async.ca.shared.global [%2+%7], [%4], %6;\n\t"
                 "cp.async.commit_group;\n\t}" ::"r"(wd), "l"(wp), "r"(sd), "l"(sp), "l"(zp), "r"(int(on)), "n"(SB), "n"(32 * SB)
                 : "memory");
  } else if constexpr (!HAS_ZERO && TWO) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t" MGV_LEAN_W
                 "@q cp.async.ca.shared.global [%2], [%3], %6;\n\t"
                 "@q cp.async.ca.shared.global [%2+%7], [%4], %6;\n\t"
                 "cp.async.commit_group;\n\t}" ::"r"(wd), "l"(wp), "r"(sd), "l"(sp), "l"(sp + n_cols), "r"(int(on)), "n"(SB), "n"(32 * SB)
                 : "memory");
  } else {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %7, 0;\n\t" MGV_LEAN_W
                 "@q cp.async.ca.shared.global [%2], [%3], %8;\n\t"
                 "@q cp.async.ca.shared.global [%2+%9], [%4], %8;\n\t"
                 "@q cp.async.ca.shared.global [%2+%10], [%5], %8;\n\t"
                 "@q cp.async.ca.shared.global [%2+%11], [%6], %8;\n\t"
                 "cp.async.commit_group;\n\t}" ::"r"(wd), "l"(wp), "r"(sd), "l"(sp), "l"(sp + n_cols), "l"(zp), "l"(zp + n_cols),
                 "r"(int(on)), "n"(SB), "n"(32 * SB), "n"(64 * SB), "n"(96 * SB)
                 : "memory");
  }
}
#undef MGV_LEAN_W

// Arithmetic of one item of the steady-state kernel, 4-bit weights.  wa, sa: the lane's
// weights and scales in the slot; tab: the lane's table entry of the item; xs: the lane's x.
template <bool HAS_ZERO, bool TWO>
__device__ __forceinline__ void lean_compute4(uint32_t wa, uint32_t sa, uint32_t tab, uint32_t xs, float (&acc)[8]) {
  constexpr int SB = 8, ZO = (TWO ? 64 : 32) * SB;
  static_for<0, TWO ? 2 : 1>([&](auto h_c) {
    constexpr int H = decltype(h_c)::value;
    constexpr int ST0 = TWO ? 2 * H : 0, ST1 = TWO ? 2 * H + 2 : 4;
    // both row pairs start from the correction {c0, c1, c0, c1} of the lane's two batch columns
    const uint4 i0 = lds128_at<H * 128>(tab), i1 = lds128_at<H * 128>(tab);
    float ci[2][4] = {{__uint_as_float(i0.x), __uint_as_float(i0.y), __uint_as_float(i0.z), __uint_as_float(i0.w)},
                      {__uint_as_float(i1.x), __uint_as_float(i1.y), __uint_as_float(i1.z), __uint_as_float(i1.w)}};
    static_for<ST0, ST1>([&](auto st_c) {
      constexpr int ST = decltype(st_c)::value;
      const uint4 wv = lds128_at<ST * 512>(wa);
      const uint4 xv = lds128_at<ST * 64>(xs);
      uint32_t hh[4][4];
      convert_unit_raw(wv, hh);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        mma_16816(ci[q], hh[2 * q][0], hh[2 * q + 1][0], hh[2 * q][1], hh[2 * q + 1][1], xv.x, xv.y);
        mma_16816(ci[q], hh[2 * q][2], hh[2 * q + 1][2], hh[2 * q][3], hh[2 * q + 1][3], xv.z, xv.w);
      }
    });
    const uint2 sv = lds64_at<H * 32 * SB>(sa);
    const float sf[4] = {half_lo(sv.x), half_hi(sv.x), half_lo(sv.y), half_hi(sv.y)};
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[q * 4 + e] = fmaf(sf[2 * q + (e >> 1)], ci[q][e], acc[q * 4 + e]);
    if constexpr (HAS_ZERO) {
      const uint2 zv = lds64_at<ZO + H * 32 * SB>(sa);
      const uint2 sx = lds64_at<H * 128 + 16>(tab);
      const float zf[4] = {half_lo(zv.x), half_hi(zv.x), half_lo(zv.y), half_hi(zv.y)};
      const float sxf[2] = {__uint_as_float(sx.x), __uint_as_float(sx.y)};
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[q * 4 + e] = fmaf(zf[2 * q + (e >> 1)], sxf[e & 1], acc[q * 4 + e]);
    }
  });
}

// The same for 8-bit weights: scaled (and shifted) in fp16 with the reference's rounding points,
// then straight into the accumulators.
template <bool HAS_ZERO, bool TWO>
__device__ __forceinline__ void lean_compute8(uint32_t wa, uint32_t sa, uint32_t xs, float (&acc)[4]) {
  constexpr int SB = 4, ZO = (TWO ? 64 : 32) * SB;
  static_for<0, TWO ? 2 : 1>([&](auto h_c) {
    constexpr int H = decltype(h_c)::value;
    constexpr int ST0 = TWO ? 2 * H : 0, ST1 = TWO ? 2 * H + 2 : 4;
    const uint32_t sv = lds32_at<H * 32 * SB>(sa);
    const uint32_t s2[2] = {dup_lo(sv), dup_hi(sv)};
    [[maybe_unused]] uint32_t z2[2] = {0u, 0u};
    if constexpr (HAS_ZERO) {
      const uint32_t zv = lds32_at<ZO + H * 32 * SB>(sa);
      z2[0] = dup_lo(zv);
      z2[1] = dup_hi(zv);
    }
    static_for<ST0, ST1>([&](auto st_c) {
      constexpr int ST = decltype(st_c)::value;
      const uint4 wv = lds128_at<ST * 512>(wa);
      const uint4 xv = lds128_at<ST * 64>(xs);
      uint32_t hh[2][4];
      convert_unit<8>(wv, hh);
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hh[r][i] = hmul2_rn(hh[r][i], s2[r]);
          if constexpr (HAS_ZERO) hh[r][i] = hadd2_rn(hh[r][i], z2[r]);
        }
      mma_16816(acc, hh[0][0], hh[1][0], hh[0][1], hh[1][1], xv.x, xv.y);
      mma_16816(acc, hh[0][2], hh[1][2], hh[0][3], hh[1][3], xv.z, xv.w);
    });
  });
}

template <int BITS, bool HAS_ZERO, bool TWO, int D, int NW>
__global__ void __launch_bounds__(NW * 32, 1) gemv_lean_kernel(const __grid_constant__ GemvParams p) {
  constexpr int THREADS = NW * 32, KI = 128, STEPS = 4;
  constexpr int RPG = Geometry<BITS>::RPG, TILE_ROWS = Geometry<BITS>::TILE_ROWS;
  constexpr int SB = RPG * 2;                                        // bytes of scales per lane and group
  constexpr int SLOT = STEPS * 512 + 32 * SB * (TWO ? 2 : 1) * (HAS_ZERO ? 2 : 1);
  constexpr int NACC = (RPG / 2) * 4;
  constexpr int EL = TWO ? KI / 16 : KI / 8;                         // lanes (chunks of 8 k) per table entry
  constexpr int TAB_ITEM = TWO ? 256 : 128;                          // table bytes per item
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float *part = reinterpret_cast<float *>(smem_raw);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int M = p.M, ipt = p.ipt;
  const int t_first = range_lo(blockIdx.x, p.deal_base, p.deal_rem);
  const int t_end = range_lo(blockIdx.x + 1, p.deal_base, p.deal_rem);
  // A launch that waits for peers counts itself in before it lets dependent launches start;
  // storing the returned value to shared memory makes thread 0 (and, behind the barrier, the
  // block) wait until the count has been performed, so no block of a later launch can be counted
  // ahead of it.  (Done after the first weight copies are on their way, see below.)
  __shared__ unsigned sh_wait_target;
  auto count_in = [&]() {
    if (threadIdx.x == 0) sh_wait_target = wait_enter(p);
    __syncthreads();
    pdl_launch_dependents();
  };
  if (!p.wait_flag) pdl_launch_dependents();
  if (t_first >= t_end) {
    if (p.wait_flag) count_in();
    pdl_wait();
    signal_peers(p);
    return;
  }


  // the lane's sources at tile 0, k = 0: row group g, chunk t
  const uint32_t group_bytes = uint32_t(p.K) * 2;  // one row group: RPG rows x K weights
  const uint32_t tile_bytes = group_bytes * RG;
  const uint8_t *wl = p.w + size_t(g) * group_bytes + t * 16;
  const __half *sl = p.scale + g * RPG;
  const __half *zl = HAS_ZERO ? p.zero + g * RPG : nullptr;
  const int gs = p.gshift < 0 ? 31 : p.gshift - 7;  // log2 of the items per group (unused with two groups per item)
  const uint32_t n_cols = uint32_t(p.N);

  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t ring = smem_base + p.ring_off + uint32_t(warp) * (D * SLOT);
  const uint32_t ring_end = ring + D * SLOT;
  const uint32_t w_lane = lane * 16, s_lane = STEPS * 512 + lane * SB;
  const uint32_t tab_lane = smem_base + p.tab_off + t * 32;
  // the lane reads batch row g of the staged x (lanes without a row read row M-1 and are ignored)
  const uint32_t xs_lane = smem_base + p.xs_off + min(g, M - 1) * p.xs_pitch + t * 16;
  const int n_out = M * TILE_ROWS, slot_floats = NW * n_out;

  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
  bool first_round = true;

  for (int ta = t_first; ta < t_end; ta += p.slots) {
    const int tb = min(t_end, ta + p.slots);
    const int n = ((tb - ta) * ipt - warp + NW - 1) / NW;  // this warp's items: warp, warp + NW, ... (ipt >= NW)
    int i_tg = ta, i_ki = warp;                            // the next item to copy
    int c_tile = 0, c_ki = warp;                           // the next item to compute (tile relative to ta)
    auto issue = [&](uint32_t slot, bool on) {
      const uint32_t woff = uint32_t(i_tg) * tile_bytes + uint32_t(i_ki) * (KI * 2);
      const uint32_t grp = TWO ? uint32_t(i_ki) * 2 : uint32_t(i_ki >> gs);
      const uint32_t soff = grp * n_cols + uint32_t(i_tg) * TILE_ROWS;
      lean_copy_item<SB, HAS_ZERO, TWO>(slot + w_lane, wl + woff, slot + s_lane, sl + soff, zl + soff, n_cols, on);
      i_ki += NW;
      if (i_ki >= ipt) { i_ki -= ipt; ++i_tg; }
    };
    int filled = 0;
    if (first_round) {
      // weights and scales do not depend on the previous kernel of the stream: the first copies
      // start before a programmatic dependent launch is released; x is read after the wait
      const int prefill = min(D, p.prefill);
      for (; filled < prefill; ++filled) issue(ring + filled * SLOT, filled < n);
      prefetch_hint(p);
      if (p.wait_flag) count_in();
      pdl_wait();
      if (p.wait_flag) wait_arrived(p, sh_wait_target);  // the peers' slices this call consumes have landed

      const int chunks = p.K / 8, stage_total = M * chunks;
      uint8_t *tabp = smem_raw + p.tab_off;
      for (int i0 = 0; i0 < stage_total; i0 += THREADS) {
        const int i = i0 + threadIdx.x;
        const int m = i / chunks, ch = i - m * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i < stage_total) v = __ldcg(reinterpret_cast<const uint4 *>(p.x + size_t(m) * p.ldx + ch * 8));
        if constexpr (BITS == 4) {
          // a chunk of 8 k is {lo lo hi hi lo lo hi hi}: the hi pairs meet the 1024+16u halves
          float lo = half_lo(v.x) + half_hi(v.x) + half_lo(v.z) + half_hi(v.z);
          float hi = half_lo(v.y) + half_hi(v.y) + half_lo(v.w) + half_hi(v.w);
#pragma unroll
          for (int o = 1; o < EL; o <<= 1) {
            lo += __shfl_xor_sync(0xffffffffu, lo, o);
            hi += __shfl_xor_sync(0xffffffffu, hi, o);
          }
          if (i < stage_total && (lane & (EL - 1)) == 0) {
            float *e = reinterpret_cast<float *>(tabp + (ch / EL) * 128 + (m >> 1) * 32) + (m & 1);
            const float c = -1032.0f * lo - 72.0f * hi;
            e[0] = c; e[2] = c; e[4] = lo + hi;
          }
          v.y = hmul2_rn(v.y, 0x2c002c00u);  // half2(1/16, 1/16); exact unless |x| < 2^-10
          v.w = hmul2_rn(v.w, 0x2c002c00u);
        }
        if (i < stage_total) *reinterpret_cast<uint4 *>(smem_raw + p.xs_off + size_t(m) * p.xs_pitch + ch * 16) = v;
      }

      __syncthreads();

      first_round = false;
    }
    for (; filled < D; ++filled) issue(ring + filled * SLOT, filled < n);

    uint32_t slot = ring;
    for (int j = 0; j < n; ++j) {
      cp_async_wait_fixed<D - 1>();  // the oldest group, i.e. this item, has landed
      if constexpr (BITS == 4)
        lean_compute4<HAS_ZERO, TWO>(slot + w_lane, slot + s_lane, tab_lane + uint32_t(c_ki) * TAB_ITEM,
                                     xs_lane + uint32_t(c_ki) * (KI * 2), acc);
      else
        lean_compute8<HAS_ZERO, TWO>(slot + w_lane, slot + s_lane, xs_lane + uint32_t(c_ki) * (KI * 2), acc);
      c_ki += NW;
      if (c_ki >= ipt) {  // the warp leaves the tile: park its sums
        flush_acc<BITS, VAR_MMA, 8>(part + size_t(c_tile) * slot_floats + warp * n_out, acc, M, g, t);
        c_ki -= ipt;
        ++c_tile;
      }
      issue(slot, j + D < n);  // refill the slot just consumed
      slot += SLOT;
      if (slot == ring_end) slot = ring;
    }
    cp_async_wait_fixed<0>();

    if (c_tile < tb - ta) flush_acc<BITS, VAR_MMA, 8>(part + size_t(c_tile) * slot_floats + warp * n_out, acc, M, g, t);
    // the epilogue's parameters and this thread's first bias value are on their way before the block meets
    const EpilogueRegs ep(p);
    const int total = (tb - ta) * n_out;
    int tile = int(threadIdx.x) / n_out, i = int(threadIdx.x) - tile * n_out;
    float b = int(threadIdx.x) < total ? ep.bias_of((ta + tile) * TILE_ROWS + i % TILE_ROWS) : 0.0f;
    __syncthreads();

    // every warp has visited every tile of the round (ipt >= NW): add the warps' sums, four chains in a fixed order
    for (int e = threadIdx.x; e < total; e += THREADS) {
      if (e != int(threadIdx.x)) {
        tile = e / n_out;
        i = e - tile * n_out;
        b = ep.bias_of((ta + tile) * TILE_ROWS + i % TILE_ROWS);
      }
      const float *src = part + size_t(tile) * slot_floats + i;
      float v4[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) v4[w] = src[w * n_out];
#pragma unroll
      for (int w = 4; w < NW; ++w) v4[w & 3] += src[w * n_out];
      ep.store<TILE_ROWS>(p, ta + tile, i, (v4[0] + v4[1]) + (v4[2] + v4[3]), b);
    }
    if (tb < t_end) __syncthreads();  // part is reused by the next round

  }
  signal_peers(p);
}

// ------------------------------------------------------------------------------------------
// launcher
// ------------------------------------------------------------------------------------------
namespace {

template <int BITS, bool HZ, bool TWO, int NW>
mgv_status launch_lean_depth(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  switch (pl.depth) {
    case 1: return launch_configured<gemv_lean_kernel<BITS, HZ, TWO, 1, NW>>(p, pl, s);
    case 2: return launch_configured<gemv_lean_kernel<BITS, HZ, TWO, 2, NW>>(p, pl, s);
    case 3: return launch_configured<gemv_lean_kernel<BITS, HZ, TWO, 3, NW>>(p, pl, s);
    case 4: return launch_configured<gemv_lean_kernel<BITS, HZ, TWO, 4, NW>>(p, pl, s);
    case 5: return launch_configured<gemv_lean_kernel<BITS, HZ, TWO, 5, NW>>(p, pl, s);
    case 6: return launch_configured<gemv_lean_kernel<BITS, HZ, TWO, 6, NW>>(p, pl, s);
    default: return fail(MGV_STATUS_CUDA_ERROR, "internal: no steady-state kernel of ring depth %d", pl.depth);
  }
}

template <int BITS, bool HZ, bool TWO>
mgv_status launch_lean_nw(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.nw == 16) return launch_lean_depth<BITS, HZ, TWO, 16>(p, pl, s);
  return fail(MGV_STATUS_CUDA_ERROR, "internal: no steady-state kernel of %d warps", pl.nw);
}

template <int BITS, bool HZ>
mgv_status launch_lean(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  return pl.two_groups ? launch_lean_nw<BITS, HZ, true>(p, pl, s) : launch_lean_nw<BITS, HZ, false>(p, pl, s);
}

}  // namespace

mgv_status launch_fast(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.bits == 4) return pl.has_zero ? launch_lean<4, true>(p, pl, s) : launch_lean<4, false>(p, pl, s);
  return pl.has_zero ? launch_lean<8, true>(p, pl, s) : launch_lean<8, false>(p, pl, s);
}

}  // namespace mgv
