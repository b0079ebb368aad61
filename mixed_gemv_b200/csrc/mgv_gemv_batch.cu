// The single-pass GEMV kernel for batches of 9..16 activation rows, K = 16 * 128 * KPW
// (K = 2048, 4096, 6144, 8192): every weight byte is read from HBM once for all rows.
//
// The reference's only answer to a batch is batch_count, one full pass over the weights per
// activation row (gemv/kernel/mixed_gemv.h:134,146-149).  Here the batch rides the N dimension of
// mma.m16n8k16 -- two fragments of eight batch columns -- so one conversion of a 16-byte weight
// unit feeds sixteen rows.  Sixteen rows of x no longer fit an SM (K = 8192: 256 KB), so x is not
// kept for the whole launch as in the M <= 8 kernel: a warp holds the two x fragments of ONE of
// its k ranges (32 registers) and uses them for a group of TG = 2 row tiles before it moves to its
// next k range; the accumulators of the group's tiles stay in registers over all k ranges.  x is
// thus read once per tile group and k range -- L2 traffic of the size of the weight stream, no HBM
// traffic.  The L2 latency of these reads is kept off the warp's path: while range J is computed
// the fragments of range J + 1 travel by cp.async into the warp's own (still unused) slots of the
// partial-sum buffer and are picked up from there; the next group's first range is requested
// before the block meets to add up the finished group.
//
// Order of a warp's items: tile group, k range J = 0..KPW-1, tile of the group.  The per-lane
// cp.async ring holds one item per tile of the group (slot = tile in group, an immediate); an
// item's slot is refilled with the same tile's next k range, or the next group's first.
#include "mgv_gemv_parts.cuh"

namespace mgv {

// One 4-bit item for both batch fragments: wa, sa, tab as in the M <= 8 kernel; xv[f][st] the
// lane's x chunk of step st for batch rows f*8 + g; acc[f][c * 4 + r] as park stores it.
template <bool HAS_ZERO, bool TWO, bool FIRST, int DOFF>
__device__ __forceinline__ void batch_compute4(uint32_t wa, uint32_t sa, uint32_t tab, const uint4 (&xv)[2][4], float (&acc)[2][8]) {
  constexpr int SB = 8, ZO = (TWO ? 64 : 32) * SB;
  static_for<0, TWO ? 2 : 1>([&](auto h_c) {
    constexpr int H = decltype(h_c)::value;
    constexpr int ST0 = TWO ? 2 * H : 0, ST1 = TWO ? 2 * H + 2 : 4;
    // table entry of group h, fragment f at tab + (h * 2 + f) * 128: {c0, c1, c0, c1, sum x0, sum x1}
    float ci[2][2][4];
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint4 i = f == 0 ? lds128_at<(H * 2) * 128>(tab) : lds128_at<(H * 2 + 1) * 128>(tab);
        ci[f][q][0] = __uint_as_float(i.x); ci[f][q][1] = __uint_as_float(i.y);
        ci[f][q][2] = __uint_as_float(i.z); ci[f][q][3] = __uint_as_float(i.w);
      }
    static_for<ST0, ST1>([&](auto st_c) {
      constexpr int ST = decltype(st_c)::value;
      const uint4 wv = lds128_at<DOFF + ST * 512>(wa);
      const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t hh[4][4];  // [row][pair]: pairs 0 and 2 hold 1024 + u, pairs 1 and 3 hold 64 + u
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const uint32_t top = wr[r] >> 8;
        asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(hh[r][0]) : "r"(wr[r]));
        asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(hh[r][1]) : "r"(wr[r]));
        asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(hh[r][2]) : "r"(top));
        asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(hh[r][3]) : "r"(top));
      }
#pragma unroll
      for (int f = 0; f < 2; ++f)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          mma_16816(ci[f][q], hh[2 * q][0], hh[2 * q + 1][0], hh[2 * q][1], hh[2 * q + 1][1], xv[f][ST].x, xv[f][ST].y);
          mma_16816(ci[f][q], hh[2 * q][2], hh[2 * q + 1][2], hh[2 * q][3], hh[2 * q + 1][3], xv[f][ST].z, xv[f][ST].w);
        }
    });
    const uint2 sv = lds64_at<DOFF + H * 32 * SB>(sa);
    const float sf[4] = {half_lo(sv.x), half_hi(sv.x), half_lo(sv.y), half_hi(sv.y)};
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float &a = acc[f][(e & 1) * 4 + 2 * q + (e >> 1)];
          if constexpr (FIRST && H == 0) a = sf[2 * q + (e >> 1)] * ci[f][q][e];
          else a = fmaf(sf[2 * q + (e >> 1)], ci[f][q][e], a);
        }
    if constexpr (HAS_ZERO) {
      const uint2 zv = lds64_at<DOFF + ZO + H * 32 * SB>(sa);
      const float zf[4] = {half_lo(zv.x), half_hi(zv.x), half_lo(zv.y), half_hi(zv.y)};
#pragma unroll
      for (int f = 0; f < 2; ++f) {
        const uint2 sx = f == 0 ? lds64_at<(H * 2) * 128 + 16>(tab) : lds64_at<(H * 2 + 1) * 128 + 16>(tab);
        const float sxf[2] = {__uint_as_float(sx.x), __uint_as_float(sx.y)};
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int c = 0; c < 2; ++c) acc[f][c * 4 + r] = fmaf(zf[r], sxf[c], acc[f][c * 4 + r]);
      }
    }
  });
}

// The same for 8-bit weights: scaled (and shifted) in fp16 with the reference's rounding points
// (gemv/warp/warp_dequantizer.h:52-59), then straight into the accumulators (the mma's own order).
template <bool HAS_ZERO, bool TWO, bool FIRST, int DOFF>
__device__ __forceinline__ void batch_compute8(uint32_t wa, uint32_t sa, const uint4 (&xv)[2][4], float (&acc)[2][4]) {
  constexpr int SB = 4, ZO = (TWO ? 64 : 32) * SB;
  static_for<0, TWO ? 2 : 1>([&](auto h_c) {
    constexpr int H = decltype(h_c)::value;
    constexpr int ST0 = TWO ? 2 * H : 0, ST1 = TWO ? 2 * H + 2 : 4;
    const uint32_t sv = lds32_at<DOFF + H * 32 * SB>(sa);
    const uint32_t s2[2] = {dup_lo(sv), dup_hi(sv)};
    [[maybe_unused]] uint32_t z2[2] = {0u, 0u};
    if constexpr (HAS_ZERO) {
      const uint32_t zv = lds32_at<DOFF + ZO + H * 32 * SB>(sa);
      z2[0] = dup_lo(zv);
      z2[1] = dup_hi(zv);
    }
    static_for<ST0, ST1>([&](auto st_c) {
      constexpr int ST = decltype(st_c)::value;
      const uint4 wv = lds128_at<DOFF + ST * 512>(wa);
      uint32_t hh[2][4];
      convert_unit<8>(wv, hh);
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hh[r][i] = hmul2_rn(hh[r][i], s2[r]);
          if constexpr (HAS_ZERO) hh[r][i] = hadd2_rn(hh[r][i], z2[r]);
        }
#pragma unroll
      for (int f = 0; f < 2; ++f) {
        if constexpr (FIRST && ST == 0) mma_16816_z(acc[f], hh[0][0], hh[1][0], hh[0][1], hh[1][1], xv[f][ST].x, xv[f][ST].y);
        else mma_16816(acc[f], hh[0][0], hh[1][0], hh[0][1], hh[1][1], xv[f][ST].x, xv[f][ST].y);
        mma_16816(acc[f], hh[0][2], hh[1][2], hh[0][3], hh[1][3], xv[f][ST].z, xv[f][ST].w);
      }
    });
  });
}

template <int BITS, bool HAS_ZERO, bool TWO, int KPW>
__global__ void __launch_bounds__(512, 1) gemv_batch_kernel(const __grid_constant__ GemvParams p) {
  constexpr int NW = 16, THREADS = 512, KI = 128, STEPS = 4, TE = TWO ? 2 : 1, TG = 2;
  constexpr int RPG = Geometry<BITS>::RPG, TILE_ROWS = Geometry<BITS>::TILE_ROWS, SB = RPG * 2, NACC = (RPG / 2) * 4;
  constexpr int SLOT = STEPS * 512 + 32 * SB * TE * (HAS_ZERO ? 2 : 1);
  constexpr int TAB_J = TE * 2 * 128;  // table bytes per k range: [group][fragment][4 lane quarters] x 32 B
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float *part = reinterpret_cast<float *>(smem_raw);  // [TG][NW][M][TILE_ROWS]

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int M = p.M;
  const int t_first = range_lo(blockIdx.x, p.deal_base, p.deal_rem);
  const int t_end = range_lo(blockIdx.x + 1, p.deal_base, p.deal_rem);
  pdl_launch_dependents();
  if (t_first >= t_end) return;  // (the host never launches more blocks than tiles)

  const uint32_t group_bytes = uint32_t(p.K) * 2, tile_bytes = group_bytes * RG;
  const uint32_t n_col_bytes = uint32_t(p.N) * 2;
  const int gs = p.gshift < 0 ? 31 : p.gshift - 7;
  const uint8_t *wl = p.w + size_t(g) * group_bytes + t * 16 + uint32_t(warp) * (KI * 2);
  const __half *sl = p.scale + g * RPG;
  uint32_t soff[KPW];  // byte offset of k range J's (first) group in the scale matrix
#pragma unroll
  for (int j = 0; j < KPW; ++j) {
    const uint32_t ki = uint32_t(warp) + uint32_t(j) * NW;
    soff[j] = (TWO ? ki * 2 : (ki >> gs)) * n_col_bytes;
  }
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t ring = smem_base + p.ring_off + uint32_t(warp) * (TG * SLOT);
  const uint32_t wa = ring + lane * 16, sa = ring + STEPS * 512 + lane * SB;
  const uint32_t tab_lane = smem_base + p.tab_off + uint32_t(warp) * (KPW * TAB_J) + t * 32;
  constexpr int PITCH = 512;  // floats between the warps' slots of a parked tile: 16 rows of x at most, 2 KB
  const int n_out = M * TILE_ROWS, slot_floats = NW * PITCH;
  // the lane's x rows: batch rows g and 8 + g (lanes without a row read row M-1 and are ignored)
  const __half *xrow[2] = {p.x + size_t(g) * p.ldx + warp * KI + t * 8, p.x + size_t(min(8 + g, M - 1)) * p.ldx + warp * KI + t * 8};

  const int ntl = t_end - t_first, n_groups = (ntl + TG - 1) / TG;
  // the lane's pointers into the first tile of the group whose items are copied
  const uint8_t *wt = wl + size_t(t_first) * tile_bytes;
  const __half *st = sl + size_t(t_first) * TILE_ROWS;
  [[maybe_unused]] const __half *zt = HAS_ZERO ? p.zero + g * RPG + size_t(t_first) * TILE_ROWS : nullptr;
  // copies k range J of tile TT of the group at (wt_, st_, zt_) into the tile's ring slot
  auto copy = [&](auto tt_c, auto j_c, const uint8_t *wt_, const __half *st_, const __half *zt_) {
    constexpr int TT = decltype(tt_c)::value, J = decltype(j_c)::value;
    tile_copy_item<SB, HAS_ZERO, TWO, TT * SLOT, J * (NW * KI * 2)>(wa, wt_ + size_t(TT) * tile_bytes, sa, ptr_plus(st_ + TT * TILE_ROWS, soff[J]),
                                                                   HAS_ZERO ? ptr_plus(zt_ + TT * TILE_ROWS, soff[J]) : nullptr, n_col_bytes);
  };
  auto commit_empty = [&]() { asm volatile("cp.async.commit_group;" ::: "memory"); };

  // the first group's first k range: weights and scales do not depend on the previous kernel
  static_for<0, TG>([&](auto tt_c) {
    constexpr int TT = decltype(tt_c)::value;
    if (TT < ntl) copy(tt_c, std::integral_constant<int, 0>{}, wt, st, zt);
    else commit_empty();
  });
  prefetch_hint(p);
  pdl_wait();

  uint4 xr[2][4];
  auto load_into = [&](uint4 (&dst)[2][4], int j) {  // straight from L2
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int s = 0; s < STEPS; ++s) dst[f][s] = __ldcg(reinterpret_cast<const uint4 *>(xrow[f] + j * (NW * KI) + s * 32));
  };
  // The warp's staging area for the x fragments of its NEXT k range: fragment f lies in the warp's
  // slot of parked tile f (2 KB each: [step][lane] 16 bytes, every lane copies what it reads).  The
  // warp parks its sums there only after its last pick-up, and the block's barrier after the
  // addition keeps the other warps' reads of it before the next group's first copy.
  const uint32_t stage = smem_base + uint32_t(warp) * (PITCH * 4) + lane * 16;
  auto stage_x = [&](int j) {
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int s = 0; s < STEPS; ++s)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage + f * (NW * PITCH * 4) + s * 512),
                     "l"(xrow[f] + j * (NW * KI) + s * 32)
                     : "memory");
  };
  auto pick_up_x = [&]() {
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int s = 0; s < STEPS; ++s) {
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(stage + f * (NW * PITCH * 4) + s * 512));
        xr[f][s] = v;
      }
  };
  // Per-warp correction table of the 4-bit kernels, built by the tensor cores as in the M <= 8
  // kernel, one pass over the warp's k ranges from the last to the first (whose fragments then stay
  // in the registers for the first tile group), the next range's loads in flight meanwhile:
  // -(1032*sum lo + 72*sum hi) and sum x per batch column, in the accumulator layout.
  if constexpr (BITS == 4) {
    uint4 xo[2][4];  // the other buffer of the pair (the accumulators are not alive yet)
    load_into((KPW - 1) % 2 == 0 ? xr : xo, KPW - 1);
    static_for<0, KPW>([&](auto jj_c) {
      constexpr int J = KPW - 1 - decltype(jj_c)::value;
      uint4 (&cur)[2][4] = J % 2 == 0 ? xr : xo;
      if constexpr (J > 0) load_into(J % 2 == 0 ? xo : xr, J - 1);
#pragma unroll
      for (int h = 0; h < TE; ++h)
#pragma unroll
        for (int f = 0; f < 2; ++f) {
          constexpr uint32_t LO = 0xe408e408u, HI = 0xd480d480u, ONE = 0x3c003c00u;  // half2 of -1032, -72, 1
          float cf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
          [[maybe_unused]] float sf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int s = (TWO ? 2 * h : 0); s < (TWO ? 2 * h + 2 : STEPS); ++s) {
            const uint4 v = cur[f][s];
            mma_16816(cf, LO, LO, HI, HI, v.x, v.y);
            mma_16816(cf, LO, LO, HI, HI, v.z, v.w);
            if constexpr (HAS_ZERO) {
              mma_16816(sf, ONE, ONE, ONE, ONE, v.x, v.y);
              mma_16816(sf, ONE, ONE, ONE, ONE, v.z, v.w);
            }
          }
          if (g == 0) {
            float *e = reinterpret_cast<float *>(smem_raw + p.tab_off + size_t(warp) * (KPW * TAB_J) + J * TAB_J + (h * 2 + f) * 128 + t * 32);
            *reinterpret_cast<float4 *>(e) = make_float4(cf[0], cf[1], cf[2], cf[3]);
            if constexpr (HAS_ZERO) *reinterpret_cast<float2 *>(e + 4) = make_float2(sf[0], sf[1]);
          }
        }
    });
    __syncwarp();
  } else {
    load_into(xr, 0);
  }

  // Copy groups of a warp, in order: per k range one for the staged x of the next range (empty
  // after the group's last range), then one refill per tile.  An item's weights were committed
  // TG + 1 groups before its turn, the staged x TG groups before its pick-up: at most TG younger
  // groups may be pending at either point.
  float acc[TG][2][NACC];
  for (int gi = 0; gi < n_groups; ++gi) {
    const int in_group = min(TG, ntl - gi * TG);          // tiles of this group
    const int in_next = min(TG, ntl - (gi + 1) * TG);     // tiles of the next one (<= 0: none)
    static_for<0, KPW>([&](auto j_c) {
      constexpr int J = decltype(j_c)::value;
      if constexpr (J + 1 < KPW) stage_x(J + 1);
      commit_empty();  // closes the group of the staged x (or an empty one)
      static_for<0, TG>([&](auto tt_c) {
        constexpr int TT = decltype(tt_c)::value;
        cp_async_wait_fixed<TG>();  // this item has landed
        if (TT < in_group) {
          if constexpr (BITS == 4) batch_compute4<HAS_ZERO, TWO, J == 0, TT * SLOT>(wa, sa, tab_lane + J * TAB_J, xr, acc[TT]);
          else batch_compute8<HAS_ZERO, TWO, J == 0, TT * SLOT>(wa, sa, xr, acc[TT]);
        }
        // refill the slot: the same tile's next k range, or the next group's first
        if constexpr (J + 1 < KPW) {
          if (TT < in_group) copy(tt_c, std::integral_constant<int, J + 1>{}, wt, st, zt);
          else commit_empty();
        } else {
          if (TT < in_next)
            copy(tt_c, std::integral_constant<int, 0>{}, wt + size_t(TG) * tile_bytes, st + TG * TILE_ROWS, HAS_ZERO ? zt + TG * TILE_ROWS : nullptr);
          else commit_empty();
        }
      });
      if constexpr (J + 1 < KPW) {
        cp_async_wait_fixed<TG>();  // the staged fragments of range J + 1 have landed
        pick_up_x();
      }
    });
    wt += size_t(TG) * tile_bytes;
    st += TG * TILE_ROWS;
    if constexpr (HAS_ZERO) zt += TG * TILE_ROWS;
    // the next group's first range: on its way while the block adds this group up
    if (gi + 1 < n_groups) load_into(xr, 0);
    // park the group's sums: part[tile in group][warp][batch row][row]
#pragma unroll
    for (int tt = 0; tt < TG; ++tt)
      if (tt < in_group) {
        float *dst = part + size_t(tt) * slot_floats + warp * PITCH;
#pragma unroll
        for (int f = 0; f < 2; ++f)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int col = f * 8 + 2 * t + c;
            if (col < M) {
              float *d = dst + col * TILE_ROWS + g * RPG;
              if constexpr (BITS == 4)
                *reinterpret_cast<float4 *>(d) = make_float4(acc[tt][f][4 * c], acc[tt][f][4 * c + 1], acc[tt][f][4 * c + 2], acc[tt][f][4 * c + 3]);
              else *reinterpret_cast<float2 *>(d) = make_float2(acc[tt][f][c], acc[tt][f][2 + c]);
            }
          }
      }
    // the epilogue's parameters and this thread's first bias value are on their way before the block meets
    const EpilogueRegs ep(p);
    const int total = in_group * n_out, tile0 = t_first + gi * TG;
    int tile = int(threadIdx.x) / n_out, i = int(threadIdx.x) - tile * n_out;
    float b = int(threadIdx.x) < total ? ep.bias_of((tile0 + tile) * TILE_ROWS + i % TILE_ROWS) : 0.0f;
    __syncthreads();
    for (int e = threadIdx.x; e < total; e += THREADS) {
      if (e != int(threadIdx.x)) {
        tile = e / n_out;
        i = e - tile * n_out;
        b = ep.bias_of((tile0 + tile) * TILE_ROWS + i % TILE_ROWS);
      }
      const float *src = part + size_t(tile) * slot_floats + i;
      float v4[4];  // four chains in a fixed order
#pragma unroll
      for (int w = 0; w < 4; ++w) v4[w] = src[w * PITCH];
#pragma unroll
      for (int w = 4; w < NW; ++w) v4[w & 3] += src[w * PITCH];
      ep.store<TILE_ROWS>(p, tile0 + tile, i, (v4[0] + v4[1]) + (v4[2] + v4[3]), b);
    }
    if (gi + 1 < n_groups) __syncthreads();  // the partial buffer is reused
  }
  cp_async_wait_fixed<0>();
}

namespace {

template <int BITS, bool HZ, bool TWO>
mgv_status launch_kpw(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  switch (pl.xreg) {
    case 1: return launch_configured<gemv_batch_kernel<BITS, HZ, TWO, 1>>(p, pl, s);
    case 2: return launch_configured<gemv_batch_kernel<BITS, HZ, TWO, 2>>(p, pl, s);
    case 3: return launch_configured<gemv_batch_kernel<BITS, HZ, TWO, 3>>(p, pl, s);
    case 4: return launch_configured<gemv_batch_kernel<BITS, HZ, TWO, 4>>(p, pl, s);
    default: return fail(MGV_STATUS_CUDA_ERROR, "internal: no batch kernel with %d k ranges per warp", pl.xreg);
  }
}

template <int BITS, bool HZ>
mgv_status launch_two(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  return pl.two_groups ? launch_kpw<BITS, HZ, true>(p, pl, s) : launch_kpw<BITS, HZ, false>(p, pl, s);
}

}  // namespace

mgv_status launch_batch(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.bits == 4) return pl.has_zero ? launch_two<4, true>(p, pl, s) : launch_two<4, false>(p, pl, s);
  return pl.has_zero ? launch_two<8, true>(p, pl, s) : launch_two<8, false>(p, pl, s);
}

}  // namespace mgv
