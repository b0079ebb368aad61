// The x-in-registers GEMV kernel with compile-time ring geometry -- the kernel of the decode
// shapes whose K is 16 * 128 * KPW (K = 2048, 4096, 6144, 8192), M <= 8, whole tiles per block.
//
// Same scheme as the other GEMV kernels (one 512-thread block per SM, 16 warps taking a tile's
// 128-k items round-robin, per-lane cp.async rings, weights through mma.m16n8k16 unscaled, the
// group's scale applied to the fp32 partial sum), arranged so that the work AROUND an item is
// nearly free, because the arithmetic phase of a call is bound by instruction issue and by the
// integer pipe, not by memory:
//   * warp w meets only the k ranges w, w+16, ... (KPW per tile); its x fragments for them stay
//     in registers for the whole launch;
//   * the ring holds DT whole tiles per warp (KPW * DT slots) and the tile loop is unrolled by
//     DT, so every shared-memory address of a slot and every source offset inside a tile is an
//     immediate of the load or copy instruction: per tile one 64-bit pointer bump;
//   * the first item of a tile writes the accumulators (no zeroing), a tile is parked with two
//     128-bit shared-memory stores per lane;
//   * the nibbles are converted with one shift and four masks per word (the reference converter's
//     masks, gemv/interleaved_numeric_conversion.h:225-298): the lo pairs become 1024 + u, the hi
//     pairs -- spliced into the mantissa of 64.0 instead of 1024.0 -- become 64 + u, both exact;
//     the offsets (1032 and 72 per weight, u = q + 8) are removed per item through a correction
//     table that the tensor cores build from the warp's x fragments.  (Measured and dropped: the
//     shift as a multiply-high to leave the integer pipe, C2 6.9 against 6.4 us; no shift at all
//     with a byte permute and a third mma per step for the cross terms, C2 7.1 us.)
//   * a launch that does not overlap its predecessor (no MGV_FLAG_PDL) gets its first ring fill by
//     tiled bulk copies (cp.async.bulk.tensor through a tensor map of the preprocessed weights, one
//     copy per slot issued by lane 0, completion on a per-slot mbarrier, bounded wait): the ten
//     copy instructions per lane of the ordinary fill cost the load/store unit 0.5 us at the very
//     start of a block.  C2 alone 7.9 -> 7.2 us, plain launches without a graph 10.2 -> 9.1 us.
//     (All weights by bulk copies: 7 - 9 % slower on every shape, the layout only offers 64-byte rows.)
#include "mgv_gemv_parts.cuh"

namespace mgv {

// ---- arithmetic of one item, 4-bit weights ------------------------------------------------
// wa, sa: the lane's weights and scales in the slot (shared addresses, slot offset DOFF as an
// immediate); tab: the lane's correction-table entry of the item; xv: the lane's x chunks of
// the four steps.  FIRST: the item opens a tile -- the accumulators are written, not added to.
// acc[c * 4 + r]: batch column 2t + c, row r of the lane's four (the order park_tile stores).
// creg: the lane's correction-table entries of the item in registers ({c0, c1, sum x0, sum x1} per
// group), or null: they are read from shared memory at tab.
template <bool HAS_ZERO, bool TWO, bool FIRST, int DOFF, bool TABREG = false>
__device__ __forceinline__ void tile_compute4(uint32_t wa, uint32_t sa, uint32_t tab, const uint4 (&xv)[4], float (&acc)[8],
                                              const float (*creg)[4] = nullptr) {
  constexpr int SB = 8, ZO = (TWO ? 64 : 32) * SB;
  static_for<0, TWO ? 2 : 1>([&](auto h_c) {
    constexpr int H = decltype(h_c)::value;
    constexpr int ST0 = TWO ? 2 * H : 0, ST1 = TWO ? 2 * H + 2 : 4;
    // both row pairs start from the correction {c0, c1, c0, c1} of the lane's two batch columns
    float ci[2][4];
    if constexpr (TABREG) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        ci[q][0] = creg[H][0]; ci[q][1] = creg[H][1]; ci[q][2] = creg[H][0]; ci[q][3] = creg[H][1];
      }
    } else {
      const uint4 i0 = lds128_at<H * 128>(tab), i1 = lds128_at<H * 128>(tab);
      ci[0][0] = __uint_as_float(i0.x); ci[0][1] = __uint_as_float(i0.y); ci[0][2] = __uint_as_float(i0.z); ci[0][3] = __uint_as_float(i0.w);
      ci[1][0] = __uint_as_float(i1.x); ci[1][1] = __uint_as_float(i1.y); ci[1][2] = __uint_as_float(i1.z); ci[1][3] = __uint_as_float(i1.w);
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
      for (int q = 0; q < 2; ++q) {
        mma_16816(ci[q], hh[2 * q][0], hh[2 * q + 1][0], hh[2 * q][1], hh[2 * q + 1][1], xv[ST].x, xv[ST].y);
        mma_16816(ci[q], hh[2 * q][2], hh[2 * q + 1][2], hh[2 * q][3], hh[2 * q + 1][3], xv[ST].z, xv[ST].w);
      }
    });
    const uint2 sv = lds64_at<DOFF + H * 32 * SB>(sa);
    const float sf[4] = {half_lo(sv.x), half_hi(sv.x), half_lo(sv.y), half_hi(sv.y)};
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float &a = acc[(e & 1) * 4 + 2 * q + (e >> 1)];
        if constexpr (FIRST && H == 0) a = sf[2 * q + (e >> 1)] * ci[q][e];
        else a = fmaf(sf[2 * q + (e >> 1)], ci[q][e], a);
      }
    if constexpr (HAS_ZERO) {
      const uint2 zv = lds64_at<DOFF + ZO + H * 32 * SB>(sa);
      const float zf[4] = {half_lo(zv.x), half_hi(zv.x), half_lo(zv.y), half_hi(zv.y)};
      float sxf[2];
      if constexpr (TABREG) {
        sxf[0] = creg[H][2]; sxf[1] = creg[H][3];
      } else {
        const uint2 sx = lds64_at<H * 128 + 16>(tab);
        sxf[0] = __uint_as_float(sx.x); sxf[1] = __uint_as_float(sx.y);
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) acc[c * 4 + r] = fmaf(zf[r], sxf[c], acc[c * 4 + r]);
    }
  });
}

// The same for 8-bit weights: scaled (and shifted) in fp16 with the reference's rounding points
// (gemv/warp/warp_dequantizer.h:52-59), then straight into the accumulators.
template <bool HAS_ZERO, bool TWO, bool FIRST, int DOFF>
__device__ __forceinline__ void tile_compute8(uint32_t wa, uint32_t sa, const uint4 (&xv)[4], float (&acc)[4]) {
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
      if constexpr (FIRST && ST == 0) mma_16816_z(acc, hh[0][0], hh[1][0], hh[0][1], hh[1][1], xv[ST].x, xv[ST].y);
      else mma_16816(acc, hh[0][0], hh[1][0], hh[0][1], hh[1][1], xv[ST].x, xv[ST].y);
      mma_16816(acc, hh[0][2], hh[1][2], hh[0][3], hh[1][3], xv[ST].z, xv[ST].w);
    });
  });
}

// A warp leaves a tile: its sums go to dst[col][row] (col: batch row, row: row of the tile).  The
// lane's RPG rows of one batch column are contiguous: one 128-bit (8-bit weights: 64-bit) store.
// 4-bit: acc[c * 4 + r]; 8-bit: the mma's own order, acc[r * 2 + c].
template <int BITS>
__device__ __forceinline__ void park_tile(float *dst, const float (&acc)[(16 / BITS / 2) * 4], int M, int g, int t) {
  constexpr int RPG = 16 / BITS, TILE_ROWS = 8 * RPG;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int col = 2 * t + c;
    if (col < M) {
      float *d = dst + col * TILE_ROWS + g * RPG;
      if constexpr (BITS == 4) *reinterpret_cast<float4 *>(d) = make_float4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]);
      else *reinterpret_cast<float2 *>(d) = make_float2(acc[c], acc[2 + c]);
    }
  }
}

// TFILL: the first ring fill travels by tiled bulk copies (launches that do not overlap their predecessor).
template <int BITS, bool HAS_ZERO, bool TWO, int KPW, int DT, bool TFILL = false>
__global__ void __launch_bounds__(512, 1) gemv_tile_kernel(const __grid_constant__ GemvParams p) {
  constexpr int NW = 16, THREADS = 512, KI = 128, STEPS = 4, TE = TWO ? 2 : 1, D = KPW * DT;
  constexpr int RPG = Geometry<BITS>::RPG, TILE_ROWS = Geometry<BITS>::TILE_ROWS, SB = RPG * 2, NACC = (RPG / 2) * 4;
  constexpr int SLOT = STEPS * 512 + 32 * SB * TE * (HAS_ZERO ? 2 : 1);
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float *part = reinterpret_cast<float *>(smem_raw);
  __shared__ unsigned sh_wait_target;

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int M = p.M;
  const int t_first = range_lo(blockIdx.x, p.deal_base, p.deal_rem);
  const int t_end = range_lo(blockIdx.x + 1, p.deal_base, p.deal_rem);
  // A launch that waits for peers counts itself in before it lets dependents start.  The count is
  // requested here, at entry, and picked up after the first ring fill has been issued: its round
  // trip (about a microsecond) then costs nothing.
  unsigned long long my_count = 0;
  if (p.wait_flag && threadIdx.x == 0) my_count = atomicAdd(p.wait_state, 1ull);
  auto count_in = [&]() {
    if (threadIdx.x == 0) sh_wait_target = unsigned((my_count / gridDim.x) * p.wait_delta);
    __syncthreads();
    pdl_launch_dependents();
  };
  if (!p.wait_flag) pdl_launch_dependents();
  if (t_first >= t_end) {  // (the host never launches more blocks than tiles)
    if (p.wait_flag) count_in();
    pdl_wait();
    signal_peers(p);
    return;
  }

  const uint32_t group_bytes = uint32_t(p.K) * 2, tile_bytes = group_bytes * RG;
  const uint32_t n_col_bytes = uint32_t(p.N) * 2;
  const int gs = p.gshift < 0 ? 31 : p.gshift - 7;
  // the lane's sources at tile 0, k range 0 of the warp: row group g, chunk t
  const uint8_t *wl = p.w + size_t(g) * group_bytes + t * 16 + uint32_t(warp) * (KI * 2);
  const __half *sl = p.scale + g * RPG;
  uint32_t soff[KPW];  // byte offset of k range J's (first) group in the scale matrix
#pragma unroll
  for (int j = 0; j < KPW; ++j) {
    const uint32_t ki = uint32_t(warp) + uint32_t(j) * NW;
    soff[j] = (TWO ? ki * 2 : (ki >> gs)) * n_col_bytes;
  }
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t ring = smem_base + p.ring_off + uint32_t(warp) * (D * SLOT);
  const uint32_t wa = ring + lane * 16, sa = ring + STEPS * 512 + lane * SB;
  const uint32_t tab_lane = smem_base + p.tab_off + uint32_t(warp) * (KPW * TE * 128) + t * 32;
  const int n_out = M * TILE_ROWS, slot_floats = NW * n_out;
  // First ring fill by tiled bulk copies (p.bar_off): lane 0 issues ONE copy per slot -- no per-lane copy
  // instructions for the load/store unit to work through at the block's start -- and the slot's first
  // use waits on its barrier.  Refills are per-lane cp.async as ever.
  constexpr bool tensor_fill = TFILL;
  [[maybe_unused]] const uint32_t bars = smem_base + p.bar_off + uint32_t(warp) * 64;
  if constexpr (tensor_fill) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < D; ++s) mbar_init(bars + 8 * s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
  }

  // the correction table in registers where it is small (two entries per lane: K = 4096 with groups
  // of 128 and more, K = 2048): no shared-memory round trip at the start, one read less per item
  constexpr bool TABREG = BITS == 4 && KPW * TE <= 2;
  [[maybe_unused]] float creg[KPW][TE][4];
  float acc[NACC];
  uint4 xr[KPW][4];
  const int ntl = t_end - t_first;
  // the lane's pointers into the tile whose items are copied next
  const uint8_t *wt = wl + size_t(t_first) * tile_bytes;
  const __half *st = sl + size_t(t_first) * TILE_ROWS;
  [[maybe_unused]] const __half *zt = HAS_ZERO ? p.zero + g * RPG + size_t(t_first) * TILE_ROWS : nullptr;
  // copies item J of the tile at (wt_, st_, zt_) into ring slot S
  auto copy = [&](auto s_c, auto j_c, const uint8_t *wt_, const __half *st_, const __half *zt_) {
    constexpr int S = decltype(s_c)::value, J = decltype(j_c)::value;
    tile_copy_item<SB, HAS_ZERO, TWO, S * SLOT, J * (NW * KI * 2)>(wa, wt_, sa, ptr_plus(st_, soff[J]),
                                                                  HAS_ZERO ? ptr_plus(zt_, soff[J]) : nullptr, n_col_bytes);
  };
  auto commit_empty = [&]() { asm volatile("cp.async.commit_group;" ::: "memory"); };
  // fills ring slots [lo, hi) with the block's first tiles (slot S holds k range S % KPW of tile S / KPW)
  auto fill = [&](int lo, int hi) {
    static_for<0, D>([&](auto s_c) {
      constexpr int S = decltype(s_c)::value, DTI = S / KPW, J = S % KPW;
      if (S >= lo && S < hi) {
        if (DTI < ntl) {
          if constexpr (tensor_fill) {
            tile_copy_scales<SB, HAS_ZERO, TWO, S * SLOT>(sa, ptr_plus(st + DTI * TILE_ROWS, soff[J]),
                                                           HAS_ZERO ? ptr_plus(zt + DTI * TILE_ROWS, soff[J]) : nullptr, n_col_bytes);
            if (lane == 0) {
              mbar_expect_tx(bars + 8 * S, STEPS * 512);
              bulk_item(ring + S * SLOT, &p.w_map, (t_first + DTI) * RG, warp * (KI * 2 / 64) + J * (NW * KI * 2 / 64), bars + 8 * S);
            }
          } else {
            copy(s_c, std::integral_constant<int, J>{}, wt + size_t(DTI) * tile_bytes, st + DTI * TILE_ROWS,
                 HAS_ZERO ? zt + DTI * TILE_ROWS : nullptr);
          }
        } else commit_empty();
      }
    });
  };
  // Weights and scales do not depend on the previous kernel of the stream: the first copies start
  // before a programmatic dependent launch is released; x is read after the wait.
  const int pf = min(D, p.prefill);
  fill(0, pf);
  if (!p.hint_late) prefetch_hint(p);
  if (p.wait_flag) count_in();
  pdl_wait();
  if (p.wait_flag) wait_arrived(p, sh_wait_target);  // the peers' slices this call consumes have landed
  {
    // the lane's x: batch row g (lanes without a row read row M-1 and are ignored), chunk t of every step
    const __half *xl = p.x + size_t(min(g, M - 1)) * p.ldx + warp * KI + t * 8;
#pragma unroll
    for (int j = 0; j < KPW; ++j)
#pragma unroll
      for (int s = 0; s < STEPS; ++s) xr[j][s] = __ldcg(reinterpret_cast<const uint4 *>(xl + j * (NW * KI) + s * 32));
  }
  fill(pf, D);
  // from here on the pointers name the tile DT ahead of the one being computed
  wt += size_t(DT) * tile_bytes;
  st += DT * TILE_ROWS;
  if constexpr (HAS_ZERO) zt += DT * TILE_ROWS;
  auto next_tile = [&]() {
    wt += tile_bytes;
    st += TILE_ROWS;
    if constexpr (HAS_ZERO) zt += TILE_ROWS;
  };
  // Per-warp correction table, by the tensor cores: an A fragment holding -1032 on the k
  // positions of the lo pairs and -72 on those of the hi pairs turns the x fragments into
  // -(1032*sum lo + 72*sum hi) per batch column -- already in the accumulator layout
  // {c(2t), c(2t+1)} x {row g, row g+8} the item loop starts from; all-ones gives sum x.
#pragma unroll
  for (int j = 0; j < (BITS == 4 ? KPW : 0); ++j)
#pragma unroll
    for (int h = 0; h < TE; ++h) {
      constexpr uint32_t LO = 0xe408e408u, HI = 0xd480d480u, ONE = 0x3c003c00u;  // half2 of -1032, -72, 1
      float cf[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int s = (TWO ? 2 * h : 0); s < (TWO ? 2 * h + 2 : STEPS); ++s) {
        const uint4 v = xr[j][s];
        mma_16816(cf, LO, LO, HI, HI, v.x, v.y);
        mma_16816(cf, LO, LO, HI, HI, v.z, v.w);
        if constexpr (HAS_ZERO) {
          mma_16816(sf, ONE, ONE, ONE, ONE, v.x, v.y);
          mma_16816(sf, ONE, ONE, ONE, ONE, v.z, v.w);
        }
      }
      if constexpr (TABREG) {  // every row of the product is the same: each lane holds the entry of its own t
        creg[j][h][0] = cf[0]; creg[j][h][1] = cf[1]; creg[j][h][2] = sf[0]; creg[j][h][3] = sf[1];
      } else if (g == 0) {
        float *e = reinterpret_cast<float *>(smem_raw + p.tab_off + (size_t(warp) * (KPW * TE) + j * TE + h) * 128 + t * 32);
        *reinterpret_cast<float4 *>(e) = make_float4(cf[0], cf[1], cf[2], cf[3]);
        if constexpr (HAS_ZERO) *reinterpret_cast<float2 *>(e + 4) = make_float2(sf[0], sf[1]);
      }
    }
  if constexpr (!TABREG) __syncwarp();
  if (p.hint_late) prefetch_hint(p);

  // ---- the block's tiles, DT at a time: slot addresses are immediates.  A warp parks a finished
  // tile in slot (tile % p.slots) of the partial buffer; when the last slot is written (or the
  // block's last tile) the block meets and adds the warps' sums in warp order.  The ring keeps
  // streaming across these meetings.
  const int slots = p.slots;
  int ps = 0;  // partial-buffer slot of the tile being computed
  // ALWAYS: every tile of the call has a successor DT further on, whose items refill the slots;
  // otherwise that is checked per tile.  (One call site per instantiation: the body is inlined
  // and the x fragments and accumulators stay in registers.)
  auto do_tile = [&](auto dt_c, auto always_c, int ti) {
    constexpr int DTI = decltype(dt_c)::value;
    constexpr bool ALWAYS = decltype(always_c)::value;
    const bool more = ALWAYS || ti + DT < ntl;
    static_for<0, KPW>([&](auto j_c) {
      constexpr int J = decltype(j_c)::value, S = DTI * KPW + J;
      cp_async_wait_fixed<D - 1>();  // the oldest group, i.e. this item, has landed
      if constexpr (tensor_fill)
        if (ti < DT) mbar_wait(bars + 8 * S, 0, p.err_word);  // ... its weights too, where they came by bulk copy
      if constexpr (BITS == 4) {
        if constexpr (TABREG) tile_compute4<HAS_ZERO, TWO, J == 0, S * SLOT, true>(wa, sa, 0u, xr[J], acc, creg[J]);
        else tile_compute4<HAS_ZERO, TWO, J == 0, S * SLOT>(wa, sa, tab_lane + J * (TE * 128), xr[J], acc);
      }
      else tile_compute8<HAS_ZERO, TWO, J == 0, S * SLOT>(wa, sa, xr[J], acc);
      if (more) copy(std::integral_constant<int, S>{}, j_c, wt, st, zt);
      else commit_empty();
    });
    if (more) next_tile();
    park_tile<BITS>(part + size_t(ps) * slot_floats + warp * n_out, acc, M, g, t);
    if (++ps == slots || (!ALWAYS && ti == ntl - 1)) {
      // the epilogue's parameters and this thread's first bias value are on their way before the block meets
      const EpilogueRegs ep(p);
      const int first_tile = t_first + ti - (ps - 1), total = ps * n_out;
      int tile = int(threadIdx.x) / n_out, i = int(threadIdx.x) - tile * n_out;
      float b = int(threadIdx.x) < total ? ep.bias_of((first_tile + tile) * TILE_ROWS + i % TILE_ROWS) : 0.0f;
      __syncthreads();
      for (int e = threadIdx.x; e < total; e += THREADS) {
        if (e != int(threadIdx.x)) {
          tile = e / n_out;
          i = e - tile * n_out;
          b = ep.bias_of((first_tile + tile) * TILE_ROWS + i % TILE_ROWS);
        }
        const float *src = part + size_t(tile) * slot_floats + i;
        float v4[4];  // four chains instead of one of sixteen additions (a fixed order all the same)
#pragma unroll
        for (int w = 0; w < 4; ++w) v4[w] = src[w * n_out];
#pragma unroll
        for (int w = 4; w < NW; ++w) v4[w & 3] += src[w * n_out];
        ep.store<TILE_ROWS>(p, first_tile + tile, i, (v4[0] + v4[1]) + (v4[2] + v4[3]), b);
      }
      if (ALWAYS || ti != ntl - 1) __syncthreads();  // the partial buffer is reused
      ps = 0;
    }
  };
  int tl = 0;
  for (; tl + 2 * DT <= ntl; tl += DT)  // whole groups of DT tiles that all have a successor DT further on
    static_for<0, DT>([&](auto dt_c) { do_tile(dt_c, std::true_type{}, tl + decltype(dt_c)::value); });
  for (; tl < ntl; tl += DT)            // the last DT .. 2 DT - 1 tiles: refills end
    static_for<0, DT>([&](auto dt_c) {
      const int ti = tl + decltype(dt_c)::value;
      if (ti < ntl) do_tile(dt_c, std::false_type{}, ti);
    });
  signal_peers(p);
}

// ------------------------------------------------------------------------------------------
// launcher
// ------------------------------------------------------------------------------------------
namespace {

template <int BITS, bool HZ, bool TWO, int KPW>
mgv_status launch_dt(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.tensor_fill) {
    if (pl.tile_dt == 1) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 1, true>>(p, pl, s);
    if constexpr (KPW <= 2) {
      if (pl.tile_dt == 2) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 2, true>>(p, pl, s);
    }
    if constexpr (KPW == 1) {
      if (pl.tile_dt == 3) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 3, true>>(p, pl, s);
      if (pl.tile_dt == 4) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 4, true>>(p, pl, s);
    }
    return fail(MGV_STATUS_CUDA_ERROR, "internal: no tile kernel with %d k ranges and %d tiles in flight", KPW, pl.tile_dt);
  }
  if (pl.tile_dt == 1) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 1>>(p, pl, s);
  if constexpr (KPW <= 2) {
    if (pl.tile_dt == 2) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 2>>(p, pl, s);
  }
  if constexpr (KPW == 1) {
    if (pl.tile_dt == 3) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 3>>(p, pl, s);
    if (pl.tile_dt == 4) return launch_configured<gemv_tile_kernel<BITS, HZ, TWO, KPW, 4>>(p, pl, s);
  }
  return fail(MGV_STATUS_CUDA_ERROR, "internal: no tile kernel with %d k ranges and %d tiles in flight", KPW, pl.tile_dt);
}

template <int BITS, bool HZ, bool TWO>
mgv_status launch_kpw(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  switch (pl.xreg) {
    case 1: return launch_dt<BITS, HZ, TWO, 1>(p, pl, s);
    case 2: return launch_dt<BITS, HZ, TWO, 2>(p, pl, s);
    case 3: return launch_dt<BITS, HZ, TWO, 3>(p, pl, s);
    case 4: return launch_dt<BITS, HZ, TWO, 4>(p, pl, s);
    default: return fail(MGV_STATUS_CUDA_ERROR, "internal: no tile kernel with %d k ranges per warp", pl.xreg);
  }
}

template <int BITS, bool HZ>
mgv_status launch_two(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  return pl.two_groups ? launch_kpw<BITS, HZ, true>(p, pl, s) : launch_kpw<BITS, HZ, false>(p, pl, s);
}

}  // namespace

mgv_status launch_tile(const GemvParams &p, const Plan &pl, cudaStream_t s) {
#ifdef MGV_TILE_ONLY_C2  // a build for experiments: the one instantiation of the int4 g128 K=4096 shape
  if (pl.bits == 4 && !pl.has_zero && !pl.two_groups && pl.xreg == 2) return launch_dt<4, false, false, 2>(p, pl, s);
  return fail(MGV_STATUS_UNSUPPORTED, "experiment build");
#else
  if (pl.bits == 4) return pl.has_zero ? launch_two<4, true>(p, pl, s) : launch_two<4, false>(p, pl, s);
  return pl.has_zero ? launch_two<8, true>(p, pl, s) : launch_two<8, false>(p, pl, s);
#endif
}

}  // namespace mgv
