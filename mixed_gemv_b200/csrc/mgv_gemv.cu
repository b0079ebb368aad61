// The fused dequantise + GEMV + reduce + epilogue kernel for sm_100a, and its launcher.
//
// It replaces the reference's device stack (gemv/kernel/mixed_gemv.h:133-254 and everything
// under gemv/threadblock, gemv/warp, gemv/thread, epilogue/threadblock) with one persistent
// kernel, one 512-thread block per SM:
//
//   * Work is cut into ITEMS: one row tile (8 row groups = 32 rows for 4-bit, 16 rows for 8-bit
//     weights) times 128 consecutive k.  Items are numbered tile-major and dealt in equal
//     contiguous ranges to the blocks, so every SM streams the same number of bytes whatever
//     N and K are (the reference launches ceil(N/64) blocks: fewer than there are SMs for
//     N = 4096).  Inside a block the sixteen warps take the items round-robin.
//   * In the preprocessed layout one 16-byte unit holds 4 (or 2) output rows x 8 consecutive k.
//     Lane (g = lane/4, t = lane%4) of a warp owns row group g and k chunk t of each 32-wide
//     step; an item is four steps.  Each lane copies ITS OWN 16-byte units, scales, zeros and
//     x chunks with cp.async into a per-warp ring of item slots in shared memory and reads them
//     back itself, so the ring needs no barrier at all -- the lane's cp.async groups order
//     everything -- and up to eight items per warp (all of a small call) are in flight at once
//     without holding registers.  (A ring filled by 1 KB cp.async.bulk copies was measured
//     six times slower: bulk copies of one SM do not overlap.)
//   * The lane converts with the LOP3/PRMT magic-number sequence.  Then:
//       - SIMT family (M <= 4): scale and zero are applied in fp16 with the reference's two
//         separate roundings (gemv/warp/warp_dequantizer.h:52-59), products are accumulated
//         with fp32 FMAs on CUDA cores (fma.rn.f32.f16, sm_100+), one accumulator pair per row
//         and batch row, and the 4 k lanes are summed by shuffles when a tile is left;
//       - MMA family (M <= 16): the lane's converted registers ARE the A fragment of
//         mma.m16n8k16 (rows g and g+8, with a k permutation shared with the x fragment); the
//         integer weights go through the tensor cores unscaled, and the group's scale is
//         applied once per item to the fp32 partial sum (and zero times the group's sum of x,
//         which a second mma with an all-ones A fragment delivers in the same layout).  That
//         is s*sum(q*x) + z*sum(x) = sum((q*s+z)*x) with fewer roundings than the reference.
//   * A warp parks its partial sums in shared memory when it moves to another tile; after the
//     block's items are done, ONE block barrier, then the per-warp partials are added in warp
//     order.  A tile whose items are spread over several blocks is combined through a scratch
//     slot per block: the last block to arrive (a per-tile counter) adds the slots in block
//     order, so the result does not depend on timing, and runs the epilogue.
//   * Epilogue: out = half(act(alpha*acc + beta*bias)), or the fp32 partial for K-split sharding.
//
// Blocks never wait for one another.  The only waits are for OTHER GPUs' arrival counts in the
// fused output exchange of sharded layers (wait_arrived), bounded to about a second.
//
// Four kernels share this scheme:
//   * gemv_kernel        (this file) everything: both families, M <= 16, ragged N and K, batched
//                        problems, all three ways of dealing the work;
//   * gemv_lean_kernel   (mgv_gemv_fast.cu) the MMA family's common decode shapes with the per-item
//                        bookkeeping cut down, x staged in shared memory: any K that is a multiple
//                        of 128 from 2048 up;
//   * gemv_tile_kernel   (mgv_gemv_tile.cu) the same for K = 2048, 4096, 6144, 8192 with each warp's
//                        x fragments in registers and every ring offset a compile-time constant --
//                        the bench kernel;
//   * gemv_batch_kernel  (mgv_gemv_batch.cu) batches of 9..16 rows in one pass over the weights.
// The host (make_plan) picks by shape; the epilogue (store_out), the exchange (signal_peers,
// wait_enter / wait_arrived) and the dependent-launch handling are common to all
// (mgv_gemv_parts.cuh).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <type_traits>

#include "mgv_gemv_parts.cuh"

namespace mgv {

// Set by a kernel whose bounded wait gave up; read and cleared by mgv_device_error_state.
__device__ int g_device_error_word;

// One ring slot holds one item of one warp:
//   [4 steps][32 lanes] 16 B   weights
//   [2 groups][32 lanes] SB    scales of the lane's rows, then the same for zeros
//   [XR][4 steps][xstep]       x: lane l < xstep/16 holds batch row l/4 (+8 per XR), chunk l%4
template <int BITS, bool HAS_ZERO, int KI>
struct Slot {
  static constexpr int STEPS = KI / 32;
  static constexpr int SB = (16 / BITS) * 2;  // bytes of scales per lane and group (8 or 4)
  static constexpr int W_BYTES = STEPS * 32 * 16;
  static constexpr int S_OFF = W_BYTES;
  static constexpr int Z_OFF = S_OFF + 2 * 32 * SB;
  static constexpr int X_OFF = Z_OFF + (HAS_ZERO ? 2 * 32 * SB : 0);
};
// Per-lane constants of the kernel, computed once.
struct LaneCtx {
  int g, t;
  uint32_t w_off;   // lane * 16: the lane's unit inside a step of a slot
  uint32_t s_off;   // S_OFF + lane * SB
  uint32_t x_off;   // X_OFF + lane * 16: where the lane's own x copies go in a slot
  int xstep;        // bytes of x per step in a slot
  bool copies_x[2]; // this lane carries batch row r*8+g into the ring
  // where the lane READS x: either its slot (x travels in the ring) or the block's staged copy
  bool staged;
  uint32_t xr_base;     // ring: offset in the slot; staged: shared address of the lane's chunk at k = 0
  uint32_t xr_step;     // bytes between steps: xstep (ring) or 64 (staged)
  uint32_t xr_frag;     // MMA: bytes from batch rows 0..7 to rows 8..15
  uint32_t xr_row;      // SIMT: bytes between batch rows
};

// Walks a warp's items (every NW-th item of the block's range) without dividing; the
// tile-dependent parts of the lane's source pointers are refreshed only when the tile changes.
template <int BITS, int NW>
struct Cursor {
  int tg, ki;            // global tile id, item index inside the tile
  int b;                 // problem of the batch the tile belongs to
  int cached_tg;         // tile the pointers below belong to
  const uint8_t *wt;     // lane's weight pointer at k = 0 of the tile
  const __half *xt;      // lane's x pointer at k = 0 (batch row g; 8 rows are added for the second fragment)
  const __half *st, *zt; // lane's scale / zero pointers at group 0 of the tile
  __device__ __forceinline__ void init(int idx, int ipt, int tiles) {
    tg = idx / ipt;
    ki = idx - tg * ipt;
    b = tg / tiles;
    cached_tg = -1;
  }
  __device__ __forceinline__ void next(int ipt, int tiles, bool batched) {
    ki += NW;
    while (ki >= ipt) {
      ki -= ipt;
      ++tg;
      if (batched) b = tg / tiles;
    }
  }
  __device__ __forceinline__ void refresh(const GemvParams &p, const LaneCtx &c) {
    if (tg == cached_tg) return;
    constexpr int RPG = Geometry<BITS>::RPG, TILE_ROWS = Geometry<BITS>::TILE_ROWS;
    cached_tg = tg;
    const int tile = tg - b * p.tiles;
    const int n0 = tile * TILE_ROWS;
    const int rg = min(c.g, (p.N - n0) / RPG - 1);  // lanes past a ragged N edge re-read the last valid row group
    wt = p.w + size_t(b) * p.bs_w + size_t(n0 / RPG + rg) * (size_t(p.K) * 2) + c.t * 16;
    xt = p.x + size_t(b) * p.bs_x + size_t(c.g) * p.ldx + c.t * 8;
    const size_t so = size_t(b) * p.bs_scale + n0 + rg * RPG;
    st = p.scale + so;
    zt = p.zero + so;
  }
};

// ---- start the asynchronous copies of one item into a ring slot ----
template <int BITS, bool HAS_ZERO, int VAR, int MB, int NW, bool FULL, int KI>
__device__ __forceinline__ void issue_item(uint32_t slot, const GemvParams &p, const LaneCtx &c, Cursor<BITS, NW> &cur,
                                           bool two_groups) {
  using S = Slot<BITS, HAS_ZERO, KI>;
  constexpr int STEPS = KI / 32;
  constexpr int XR = VAR == VAR_MMA ? MB / 8 : 1;
  cur.refresh(p, c);
  const int k0 = cur.ki * KI;
  const int nsteps = FULL ? STEPS : min(STEPS, (p.K - k0) / 32);
  const uint8_t *wp = cur.wt + k0 * 2;
  const uint32_t wd = slot + c.w_off;
#pragma unroll
  for (int st = 0; st < STEPS; ++st)
    if (FULL || st < nsteps) cp16_at<0>(wd + st * 512, wp + st * 64);
  const uint32_t soff = p.gshift >= 0 ? uint32_t(k0 >> p.gshift) * uint32_t(p.N) : 0u;  // G*N < 2^31 (checked by the host)
  const uint32_t sd = slot + c.s_off;
  cp_small_at<S::SB, 0>(sd, cur.st + soff);
  if (HAS_ZERO) cp_small_at<S::SB, S::Z_OFF - S::S_OFF>(sd, cur.zt + soff);
  if (two_groups && nsteps > STEPS / 2) {
    cp_small_at<S::SB, 32 * S::SB>(sd, cur.st + soff + p.N);
    if (HAS_ZERO) cp_small_at<S::SB, S::Z_OFF - S::S_OFF + 32 * S::SB>(sd, cur.zt + soff + p.N);
  }
  // x: lane g*4+t carries batch row g (+8 per fragment), chunk t -- unless the block staged x
  if (c.staged) return;
#pragma unroll
  for (int r = 0; r < XR; ++r) {
    const __half *xp = cur.xt + size_t(r * 8) * p.ldx + k0;
    uint32_t xd = slot + c.x_off + r * STEPS * c.xstep;
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      cp16_if(xd, xp + s * 32, c.copies_x[r] && (FULL || s < nsteps));
      xd += c.xstep;
    }
  }
}
// ---- arithmetic of one item, MMA family ----
// 4-bit weights go through the tensor cores as unscaled integers and the group's scale (and
// zero) is applied to the fp32 partial sum; with MAGIC they even keep the 1024 offset of the
// magic-number conversion, removed per item by `tab` (see build_tab).  8-bit weights are
// scaled in fp16 first with the reference's rounding points (their integer range makes the
// difference between the two orders of rounding comparable to the stated tolerance, and they
// have issue slots to spare).
// tab: shared address of this item's first table entry, [half-item][MB] float2 {corr, sum_x}.
template <int BITS, bool HAS_ZERO, int MB, bool FULL, bool MAGIC, int KI, int NACC>
__device__ __forceinline__ void compute_item_mma(uint32_t slot, const LaneCtx &c, float (&acc)[NACC], int nsteps, bool two_groups,
                                                 uint32_t tab, uint32_t xs) {
  using S = Slot<BITS, HAS_ZERO, KI>;
  constexpr int STEPS = KI / 32;
  constexpr int RPG = Geometry<BITS>::RPG;
  constexpr int XR = MB / 8, Q = RPG / 2;
  constexpr bool POST = BITS == 4;
  static_assert(!MAGIC || POST, "the offset trick belongs to the post-scaled 4-bit path");
  constexpr uint32_t ONES = 0x3c003c00u;       // half2(1, 1)
  constexpr int ZD = S::Z_OFF - S::S_OFF;
  const uint32_t wa = slot + c.w_off, sa = slot + c.s_off;
  float ci[XR][Q][4], cx[XR][4];
  if constexpr (POST) {
#pragma unroll
    for (int r = 0; r < XR; ++r)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        cx[r][e] = 0.0f;
#pragma unroll
        for (int q = 0; q < Q; ++q) ci[r][q][e] = 0.0f;
      }
  }
  // POST: fold the finished group into the accumulators, acc += s_row*sum(q*x) + z_row*sum(x)
  auto fold = [&](bool second) {
    uint32_t sv[RPG / 2], zv[RPG / 2];
    if (second) {
      load_rows<BITS, 32 * S::SB>(sa, sv);
      if constexpr (HAS_ZERO) load_rows<BITS, ZD + 32 * S::SB>(sa, zv);
    } else {
      load_rows<BITS, 0>(sa, sv);
      if constexpr (HAS_ZERO) load_rows<BITS, ZD>(sa, zv);
    }
    float sf[RPG], zf[RPG];
#pragma unroll
    for (int w = 0; w < RPG / 2; ++w) {
      sf[2 * w] = half_lo(sv[w]); sf[2 * w + 1] = half_hi(sv[w]);
      if constexpr (HAS_ZERO) { zf[2 * w] = half_lo(zv[w]); zf[2 * w + 1] = half_hi(zv[w]); }
    }
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      float corr[2] = {0.0f, 0.0f}, sx[2] = {cx[r][0], cx[r][1]};
      if constexpr (MAGIC) {
        // entries of batch columns 2t and 2t+1 of fragment r: {corr, sum_x} each.  Fast kernels
        // (FULL) keep one entry per item; generic ones keep one per 64 k and add the two when the
        // item is one group.
        const uint4 tv = lds128_at<0>(tab + (second ? MB * 8 : 0) + (r * 8 + 2 * (c.t)) * 8);
        corr[0] = __uint_as_float(tv.x); sx[0] = __uint_as_float(tv.y);
        corr[1] = __uint_as_float(tv.z); sx[1] = __uint_as_float(tv.w);
        if constexpr (!FULL) {
          if (!two_groups) {
            const uint4 t2 = lds128_at<0>(tab + MB * 8 + (r * 8 + 2 * (c.t)) * 8);
            corr[0] += __uint_as_float(t2.x); sx[0] += __uint_as_float(t2.y);
            corr[1] += __uint_as_float(t2.z); sx[1] += __uint_as_float(t2.w);
          }
        }
      }
#pragma unroll
      for (int q = 0; q < Q; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float &a = acc[(r * Q + q) * 4 + e];
          a = fmaf(sf[2 * q + (e >> 1)], ci[r][q][e] + corr[e & 1], a);
          if constexpr (HAS_ZERO) a = fmaf(zf[2 * q + (e >> 1)], sx[e & 1], a);
          ci[r][q][e] = 0.0f;
        }
      if constexpr (HAS_ZERO && !MAGIC) {
#pragma unroll
        for (int e = 0; e < 4; ++e) cx[r][e] = 0.0f;
      }
    }
  };
  uint32_t s2[RPG], z2[RPG];  // !POST: the current group's scales and zeros, duplicated to half2
  auto load_group = [&](bool second) {
    uint32_t sv[RPG / 2], zv[RPG / 2];
    if (second) {
      load_rows<BITS, 32 * S::SB>(sa, sv);
      if constexpr (HAS_ZERO) load_rows<BITS, ZD + 32 * S::SB>(sa, zv);
    } else {
      load_rows<BITS, 0>(sa, sv);
      if constexpr (HAS_ZERO) load_rows<BITS, ZD>(sa, zv);
    }
    dup_rows(sv, s2);
    if constexpr (HAS_ZERO) dup_rows(zv, z2);
  };
  if constexpr (!POST) load_group(false);
  auto step = [&](uint4 wv) {
    uint32_t hh[RPG][4];
    if constexpr (MAGIC) convert_unit_raw(wv, hh); else convert_unit<BITS>(wv, hh);
    if constexpr (!POST) {
#pragma unroll
      for (int r = 0; r < RPG; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hh[r][i] = hmul2_rn(hh[r][i], s2[r]);
          if constexpr (HAS_ZERO) hh[r][i] = hadd2_rn(hh[r][i], z2[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      // lanes whose batch column does not exist read bytes nobody wrote: their B column only
      // feeds output columns that are never stored
      // (MAGIC: the staged x already carries x/16 on the pairs that meet 1024+16u)
      const uint4 xv = lds128_at<0>(xs + r * c.xr_frag);
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        float(&d)[4] = *reinterpret_cast<float(*)[4]>(POST ? &ci[r][q][0] : &acc[(r * Q + q) * 4]);
        mma_16816(d, hh[2 * q][0], hh[2 * q + 1][0], hh[2 * q][1], hh[2 * q + 1][1], xv.x, xv.y);
        mma_16816(d, hh[2 * q][2], hh[2 * q + 1][2], hh[2 * q][3], hh[2 * q + 1][3], xv.z, xv.w);
      }
      if constexpr (POST && HAS_ZERO && !MAGIC) {  // every row of this product is the sum of x over the step's k
        mma_16816(cx[r], ONES, ONES, ONES, ONES, xv.x, xv.y);
        mma_16816(cx[r], ONES, ONES, ONES, ONES, xv.z, xv.w);
      }
    }
    xs += c.xr_step;
  };
#pragma unroll
  for (int st = 0; st < STEPS; ++st) {
    if (st == STEPS / 2 && two_groups) {
      if constexpr (POST) fold(false); else if (FULL || st < nsteps) load_group(true);
    }
    if (FULL || st < nsteps) step(lds128_at<0>(wa + st * 512));
  }
  if constexpr (POST) {
    if (!two_groups) fold(false);
    else if (FULL || nsteps > STEPS / 2) fold(true);  // a ragged last item has no second group
  }
}

// ---- arithmetic of one item, SIMT family: the reference's rounding points ----
template <int BITS, bool HAS_ZERO, int MB, bool FULL, int KI, int NACC>
__device__ __forceinline__ void compute_item_simt(uint32_t slot, const LaneCtx &c, float (&acc)[NACC], int nsteps, bool two_groups,
                                                  int M, uint32_t xs) {
  using S = Slot<BITS, HAS_ZERO, KI>;
  constexpr int STEPS = KI / 32;
  constexpr int RPG = Geometry<BITS>::RPG;
  constexpr int ZD = S::Z_OFF - S::S_OFF;
  const uint32_t wa = slot + c.w_off, sa = slot + c.s_off;
  uint32_t s2[RPG], z2[RPG];
  auto load_group = [&](bool second) {
    uint32_t sv[RPG / 2], zv[RPG / 2];
    if (second) {
      load_rows<BITS, 32 * S::SB>(sa, sv);
      if constexpr (HAS_ZERO) load_rows<BITS, ZD + 32 * S::SB>(sa, zv);
    } else {
      load_rows<BITS, 0>(sa, sv);
      if constexpr (HAS_ZERO) load_rows<BITS, ZD>(sa, zv);
    }
    dup_rows(sv, s2);
    if constexpr (HAS_ZERO) dup_rows(zv, z2);
  };
  load_group(false);
  auto step = [&](uint4 wv) {
    uint32_t hh[RPG][4];
    convert_unit<BITS>(wv, hh);
#pragma unroll
    for (int r = 0; r < RPG; ++r)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        hh[r][i] = hmul2_rn(hh[r][i], s2[r]);                          // half(q) * scale, rounded
        if constexpr (HAS_ZERO) hh[r][i] = hadd2_rn(hh[r][i], z2[r]);  // + zero, rounded again
      }
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (MB == 1 || m < M) {
        const uint4 xv = lds128_at<0>(xs + m * c.xr_row);
#pragma unroll
        for (int r = 0; r < RPG; ++r) {
          float &lo = acc[(m * RPG + r) * 2], &hi = acc[(m * RPG + r) * 2 + 1];
          fma_mixed(hh[r][0], xv.x, lo, hi);
          fma_mixed(hh[r][1], xv.y, lo, hi);
          fma_mixed(hh[r][2], xv.z, lo, hi);
          fma_mixed(hh[r][3], xv.w, lo, hi);
        }
      }
    }
    xs += c.xr_step;
  };
#pragma unroll
  for (int st = 0; st < STEPS; ++st) {
    if (st == STEPS / 2 && two_groups && (FULL || st < nsteps)) load_group(true);
    if (FULL || st < nsteps) step(lds128_at<0>(wa + st * 512));
  }
}
// NW warps per block: 32 where the lane state fits 64 registers (more warps hide the fixed
// latencies of the convert -> mma chains), 16 otherwise.
// GENERIC = false: K is a multiple of 128 and an item holds one group, so the item code is
// straight-line; GENERIC = true also handles a ragged last item and group size 64.
template <int BITS, bool HAS_ZERO, int VAR, int MB, int NW, bool MAGIC, bool GENERIC, int KI>
__global__ void __launch_bounds__(NW * 32, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
  constexpr int NWARP = NW, THREADS = NW * 32;
  using Geo = Geometry<BITS>;
  constexpr int RPG = Geo::RPG;
  constexpr int TILE_ROWS = Geo::TILE_ROWS;
  constexpr int NACC = VAR == VAR_MMA ? (MB / 8) * (RPG / 2) * 4 : MB * RPG * 2;
  static_assert(VAR == VAR_SIMT || MB % 8 == 0, "MMA family covers 8 or 16 batch columns");
  using S = Slot<BITS, HAS_ZERO, KI>;
  constexpr int STEPS = KI / 32;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float *part = reinterpret_cast<float *>(smem_raw);  // [slots][NWARP][M][TILE_ROWS]
  __shared__ int sh_last[2];
  __shared__ float pair_sums[512];  // pair mode: this block's sums of the tile it shares with its peer

  // the shuffle makes the warp index provably warp-uniform: branches on it need no reconvergence
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int cta = blockIdx.x;
  const int M = p.M, ipt = p.ipt;
  const int slot_floats = NWARP * M * TILE_ROWS;

  int i_begin, i_end;
  int pair_tile = -1;  // pair mode: the tile this block shares with the other block of its cluster
  if (p.align_tiles == 2) {
    // blocks 2q and 2q+1 form a cluster; the pair owns whole tiles and its items are halved
    const int pair = cta >> 1, rank = cta & 1;
    const int p0 = range_lo(pair, p.deal_base, p.deal_rem) * ipt, p1 = range_lo(pair + 1, p.deal_base, p.deal_rem) * ipt;
    const int mid = p0 + (p1 - p0 + 1) / 2;
    i_begin = rank ? mid : p0;
    i_end = rank ? p1 : mid;
    if (mid % ipt != 0 && mid < p1) pair_tile = mid / ipt;
  } else if (p.align_tiles) {
    i_begin = range_lo(cta, p.deal_base, p.deal_rem) * ipt;
    i_end = range_lo(cta + 1, p.deal_base, p.deal_rem) * ipt;
  } else {
    i_begin = range_lo(cta, p.deal_base, p.deal_rem);
    i_end = range_lo(cta + 1, p.deal_base, p.deal_rem);
  }
  // The launch counts itself in before it lets dependent launches start; storing the returned
  // value to shared memory makes thread 0 (and, behind the barrier, the block) wait until the
  // count has been performed, so no block of a later launch can be counted ahead of it.
  __shared__ unsigned sh_wait_target;
  if (p.wait_flag) {
    if (threadIdx.x == 0) sh_wait_target = wait_enter(p);
    __syncthreads();
  }
  const unsigned wait_target = p.wait_flag ? sh_wait_target : 0u;
  pdl_launch_dependents();
  // (in pair mode a block without items has no shared tile either: nobody waits for it)
  if (i_begin >= i_end) {  // (the host never launches more blocks than there is work)
    pdl_wait();
    signal_peers(p);
    return;
  }

  const int t_first = i_begin / ipt, t_last = (i_end - 1) / ipt;

  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;

  LaneCtx lc;
  lc.g = g; lc.t = t;
  lc.w_off = lane * 16;
  lc.s_off = S::S_OFF + lane * S::SB;
  lc.x_off = S::X_OFF + lane * 16;
  lc.xstep = p.xstep;
  lc.copies_x[0] = g < M;
  lc.copies_x[1] = 8 + g < M;
  lc.staged = p.xs_off >= 0;
  static_assert(!MAGIC || VAR == VAR_MMA, "the offset trick belongs to the MMA family");
  if (lc.staged) {
    // MMA: the lane reads batch row g (clamped: lanes without a row read row M-1 and are ignored)
    const int row = VAR == VAR_MMA ? min(g, M - 1) : 0;
    lc.xr_base = smem_u32(smem_raw) + p.xs_off + row * p.xs_pitch + t * 16;
    lc.xr_step = 64;
    lc.xr_frag = (8 + g < M ? 8 : 0) * p.xs_pitch;
    lc.xr_row = p.xs_pitch;
  } else {
    lc.xr_base = VAR == VAR_MMA ? lc.x_off : S::X_OFF + t * 16;
    lc.xr_step = p.xstep;
    lc.xr_frag = STEPS * p.xstep;
    lc.xr_row = 64;
  }
  const bool full_k = !GENERIC || p.K % KI == 0;  // every item has all four steps
  const bool two_groups = GENERIC && p.two_groups != 0;
  const bool batched = p.total_tiles != p.tiles;
  constexpr int TE = GENERIC ? 2 : 1;  // correction-table entries per item: per 64 k when a group can be 64 wide
  const int D = p.depth, slot_bytes = p.slot_bytes;
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t ring = smem_base + p.ring_off + uint32_t(warp) * D * slot_bytes;
  const uint32_t ring_end = ring + D * slot_bytes;
  const uint32_t tab_base = smem_base + p.tab_off;
  bool staged_done = false, waited = false;

  // ---- rounds of at most p.slots tiles ----
  for (int ta = t_first; ta <= t_last; ta += p.slots) {
    const int tb = min(t_last + 1, ta + p.slots);  // tiles [ta, tb) this round
    const int r_begin = max(i_begin, ta * ipt), r_end = min(i_end, tb * ipt);
    // this warp's items of the round: r_begin + warp, + NWARP, ...
    int n_issue = (r_end - r_begin - warp + NWARP - 1) / NWARP;
    if (n_issue < 0) n_issue = 0;
    int n_compute = n_issue;
    Cursor<BITS, NW> icur, ccur;
    icur.init(r_begin + warp, ipt, p.tiles);
    ccur = icur;
    auto issue = [&](uint32_t slot) {
      if (full_k) issue_item<BITS, HAS_ZERO, VAR, MB, NW, true, KI>(slot, p, lc, icur, two_groups);
      else if constexpr (GENERIC) issue_item<BITS, HAS_ZERO, VAR, MB, NW, false, KI>(slot, p, lc, icur, two_groups);
      icur.next(ipt, p.tiles, batched);
      --n_issue;
    };
    // Block-wide staging of x (and, MAGIC, of the correction table), first round only.  The
    // memory system serves requests in order, so the first chunks of x are requested before the
    // bulk of the ring is filled (behind it they would wait for ~200 KB of weights).
    constexpr int PRE = 2;  // chunks of x per thread fetched ahead of the ring fill
    uint4 xpre[PRE];
    const int chunks = p.K / 8, stage_total = (lc.staged && !staged_done) ? p.batch * M * chunks : 0;
    auto x_chunk = [&](int i) {
      const int bm = i / chunks, ch = i - bm * chunks;
      const int b = bm / M, m = bm - b * M;
      return __ldcg(reinterpret_cast<const uint4 *>(p.x + size_t(b) * p.bs_x + size_t(m) * p.ldx + ch * 8));
    };
    // Start one item per warp now; the rest of the ring is filled after the barrier below.  (The
    // hardware caps the bytes an SM has in flight, so filling the whole ring here would hold every
    // warp until most of it has arrived, and the arithmetic could not overlap the stream.)
    // Weights and scales do not depend on the previous kernel of the stream, x does: under a
    // programmatic dependent launch the first weight copies start before that kernel has finished.
    if (!waited && !lc.staged) {  // x travels with the weights here
      pdl_wait();
      if (p.wait_flag) wait_arrived(p, wait_target);
      waited = true;
    }
    const int prefill = min(D, p.prefill);
    for (int d = 0; d < prefill; ++d) {
      if (n_issue > 0) issue(ring + d * slot_bytes);
      cp_async_commit();
    }
    if (!waited) {
      pdl_wait();
      if (p.wait_flag) wait_arrived(p, wait_target);
      waited = true;
    }
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
      const int i = j * THREADS + threadIdx.x;
      xpre[j] = i < stage_total ? x_chunk(i) : make_uint4(0, 0, 0, 0);
    }

    // zero the partial buffer: a warp may never visit some tile of the round
    for (int i = threadIdx.x; i < (tb - ta) * slot_floats; i += THREADS) part[i] = 0.0f;
    if (stage_total > 0) {
      // Copy x to shared memory.  MAGIC kernels store x/16 on the pairs that meet the 1024+16u
      // halves (a chunk of 8 k is {lo lo hi hi lo lo hi hi}; exact unless |x| < 2^-10) and build,
      // per table entry (half an item or an item; one lane per chunk of 8 k) and batch column, the correction
      // -(1032*sum of x on the lo pairs + 72*sum on the hi pairs) and the plain sum of x.
      float2 *tab = reinterpret_cast<float2 *>(smem_raw + p.tab_off);
      for (int i0 = 0, j = 0; i0 < stage_total; i0 += THREADS, ++j) {
        const int i = i0 + threadIdx.x;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (j == 0) v = xpre[0];
        else if (j == 1) v = xpre[1];
        else if (i < stage_total) v = x_chunk(i);
        const int bm = i / chunks, ch = i - bm * chunks;
        if constexpr (MAGIC) {
          float lo = half_lo(v.x) + half_hi(v.x) + half_lo(v.z) + half_hi(v.z);
          float hi = half_lo(v.y) + half_hi(v.y) + half_lo(v.w) + half_hi(v.w);
          // lanes per table entry: half an item in generic kernels, a whole item otherwise
          constexpr int EL = GENERIC ? KI / 16 : KI / 8;
#pragma unroll
          for (int o = 1; o < EL; o <<= 1) {
            lo += __shfl_xor_sync(0xffffffffu, lo, o);
            hi += __shfl_xor_sync(0xffffffffu, hi, o);
          }
          if (i < stage_total && (lane & (EL - 1)) == 0) {
            const int b = bm / M, m = bm - b * M;
            tab[(size_t(b) * (ipt * TE) + ch / EL) * MB + m] = make_float2(-1032.0f * lo - 72.0f * hi, lo + hi);
          }
          v.y = hmul2_rn(v.y, 0x2c002c00u);  // half2(1/16, 1/16)
          v.w = hmul2_rn(v.w, 0x2c002c00u);
        }
        if (i < stage_total)
          *reinterpret_cast<uint4 *>(smem_raw + p.xs_off + size_t(bm) * p.xs_pitch + ch * 16) = v;
      }
      if constexpr (MAGIC) {
        if (p.K % KI)  // the last item has one half only: its second entry must read as zero
          for (int i = threadIdx.x; i < p.batch * MB; i += THREADS)
            tab[(size_t(i / MB) * (ipt * TE) + ipt * TE - 1) * MB + i % MB] = make_float2(0.0f, 0.0f);
      }
      staged_done = true;
    }
    __syncthreads();

    for (int d = prefill; d < D; ++d) {  // one group per slot, empty groups keep the count uniform
      if (n_issue > 0) issue(ring + d * slot_bytes);
      cp_async_commit();
    }

    {
      int cur_tile = -1;
      uint32_t slot = ring;
      while (n_compute > 0) {
        cp_async_wait_pending(D - 1);  // the oldest group, i.e. this item, has landed
        if (ccur.tg != cur_tile) {
          if (cur_tile >= 0)
            flush_acc<BITS, VAR, MB>(part + size_t(cur_tile - ta) * slot_floats + warp * M * TILE_ROWS, acc, M, g, t);
          cur_tile = ccur.tg;
        }
        if constexpr (VAR == VAR_MMA) {
          // table entry of this item: [batch][half item][MB]
          const int b = ccur.b;
          const uint32_t tab = tab_base + uint32_t((b * ipt + ccur.ki) * (TE * MB)) * 8;
          const uint32_t xs = lc.staged ? lc.xr_base + b * M * p.xs_pitch + ccur.ki * (KI * 2) : slot + lc.xr_base;
          if (full_k) compute_item_mma<BITS, HAS_ZERO, MB, true, MAGIC, KI>(slot, lc, acc, STEPS, two_groups, tab, xs);
          else if constexpr (GENERIC)
            compute_item_mma<BITS, HAS_ZERO, MB, false, MAGIC, KI>(slot, lc, acc, min(STEPS, (p.K - ccur.ki * KI) / 32), two_groups, tab, xs);
        } else {
          __syncwarp();  // x chunks are read across lanes: every lane's copies of this item have landed
          const int b = ccur.b;
          const uint32_t xs = lc.staged ? lc.xr_base + b * M * p.xs_pitch + ccur.ki * (KI * 2) : slot + lc.xr_base;
          if (full_k) compute_item_simt<BITS, HAS_ZERO, MB, true, KI>(slot, lc, acc, STEPS, two_groups, M, xs);
          else if constexpr (GENERIC)
            compute_item_simt<BITS, HAS_ZERO, MB, false, KI>(slot, lc, acc, min(STEPS, (p.K - ccur.ki * KI) / 32), two_groups, M, xs);
          __syncwarp();  // ... and are all consumed before the slot is refilled
        }
        ccur.next(ipt, p.tiles, batched);
        --n_compute;
        if (n_issue > 0) issue(slot);  // refill the slot just consumed
        cp_async_commit();
        slot += slot_bytes;
        if (slot == ring_end) slot = ring;
      }
      cp_async_wait_pending(0);

      if (cur_tile >= 0)
        flush_acc<BITS, VAR, MB>(part + size_t(cur_tile - ta) * slot_floats + warp * M * TILE_ROWS, acc, M, g, t);
    }
    __syncthreads();


    // ---- combine the warps' partials per tile; whole tiles go out, split tiles to scratch ----
    const int n_out = M * TILE_ROWS;  // at most 512: one pass of the block
    int n_partial = 0;
    int partial_tile[2], partial_first[2], partial_last[2];
    for (int tg = ta; tg < tb; ++tg) {
      const int tile_i0 = tg * ipt;
      const bool whole = i_begin <= tile_i0 && tile_i0 + ipt <= i_end;
      const float *src = part + size_t(tg - ta) * slot_floats;
      float *slot = nullptr;
      if (!whole && tg == pair_tile) {
        // shared with the peer block of the cluster: keep the sums in shared memory for the exchange below
        for (int i = threadIdx.x; i < n_out; i += THREADS) {
          float v = 0.0f;
#pragma unroll
          for (int w = 0; w < NWARP; ++w) v += src[w * n_out + i];
          pair_sums[i] = v;
        }
        continue;
      }
      if (!whole) {
        const int which = (i_begin / ipt == tg) ? 0 : 1;  // 0: the tile this block's range starts in
        slot = p.ws_slots + (size_t(cta) * 2 + which) * kSlotFloats;
        partial_tile[n_partial] = tg;
        partial_first[n_partial] = range_owner(tile_i0, p.deal_base, p.deal_rem);
        partial_last[n_partial] = range_owner(tile_i0 + ipt - 1, p.deal_base, p.deal_rem);
        ++n_partial;
      }
      for (int i = threadIdx.x; i < n_out; i += THREADS) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) v += src[w * n_out + i];
        if (whole) store_out<TILE_ROWS>(p, tg, i, v);
        else __stcg(slot + i, v);
      }
    }
    if (n_partial) {
      // Count this block's arrival on each split tile; the last arrival adds the slots in block
      // order.  Only the threads that wrote slot values fence (one warp for M = 1).
      if (threadIdx.x < n_out) __threadfence();
      __syncthreads();

      if (threadIdx.x < n_partial) {
        const int tg = partial_tile[threadIdx.x];
        const int prev = atomicAdd(p.ws_counters + tg, 1);
        const int last = prev == partial_last[threadIdx.x] - partial_first[threadIdx.x];
        if (last) p.ws_counters[tg] = 0;  // leave the scratch ready for the next launch
        sh_last[threadIdx.x] = last;
      }
      __syncthreads();
      for (int k = 0; k < n_partial; ++k) {
        if (!sh_last[k]) continue;
        const int tg = partial_tile[k];
        for (int i = threadIdx.x; i < n_out; i += THREADS) {
          __threadfence();
          float v = 0.0f;
          for (int c = partial_first[k]; c <= partial_last[k]; ++c) {
            // block c's slot for this tile: 0 if the tile is where its range starts, else 1
            const int wc = (range_lo(c, p.deal_base, p.deal_rem) / ipt == tg) ? 0 : 1;
            v += __ldcg(p.ws_slots + (size_t(c) * 2 + wc) * kSlotFloats + i);
          }
          store_out<TILE_ROWS>(p, tg, i, v);
        }
      }
    }
    if (tb <= t_last) __syncthreads();  // part and sh_last are reused by the next round

  }
  if (pair_tile >= 0) {
    // Both blocks of the cluster hold their share of the tile in pair_sums.  After a cluster
    // barrier the first block adds the two (own share first: a fixed order) through distributed
    // shared memory and runs the epilogue; a second barrier keeps the peer's memory alive until then.
    cluster_sync_all();
    if ((cta & 1) == 0)
      for (int i = threadIdx.x; i < M * TILE_ROWS; i += THREADS)
        store_out<TILE_ROWS>(p, pair_tile, i, pair_sums[i] + ld_peer_shared(&pair_sums[i], 1));
    cluster_sync_all();
  }
  signal_peers(p);
}
// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

struct DeviceInfo {
  int sms = 0;
  int cluster_pairs = 0;  // clusters of two 512-thread blocks with full shared memory that can be resident at once
  int smem_optin = 0;
  int *err_word = nullptr;
};


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
    {
      // how many clusters of two full-size blocks fit the device at once (0 if clusters cannot launch)
      auto kern = gemv_kernel<4, false, VAR_MMA, 8, 16, true, false, 128>;
      cudaFuncAttributes fa;
      int n = 0;
      if (cudaFuncGetAttributes(&fa, kern) == cudaSuccess &&
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, d.smem_optin - int(fa.sharedSizeBytes)) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(d.sms / 2 * 2);
        cfg.blockDim = dim3(512);
        cfg.dynamicSmemBytes = size_t(d.smem_optin - int(fa.sharedSizeBytes));
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
      }
      (void)cudaGetLastError();
      d.cluster_pairs = n;
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

// Overrides of the planner's choices.  The shipped library never reads the environment: these
// come from the `hints` member of the arguments (tests use it to reach every code path) and,
// only in a build with -DMGV_TUNING, from MGV_* environment variables read once per process.
struct Tuning {
  int deal = 0;        // MGV_HINT_DEAL_*
  int item = 0;        // 128 or 256
  int kernel = 0;      // MGV_HINT_KERNEL_* >> 4
  int depth = 0;       // ring depth of the staged steady-state kernel
  int dt = 0;          // tiles in flight of the x-in-registers kernel
  int hint_late = 0;   // prefetch hint after x has arrived
  long long hint_cap = 0;  // upper bound of the bytes a call prefetches for the next (0: none)
  int prefill = -1;    // ring slots filled before the wait for the previous kernel
  int one_launch = 0;  // never split a batch of 9..16 rows into two launches
  int tensor_fill = -1;  // x-in-registers kernel: 1 the first ring fill by tiled bulk copies
};

const Tuning &env_tuning() {
  static const Tuning t = [] {
    Tuning v;
#ifdef MGV_TUNING
    auto num = [](const char *name, int dflt) {
      const char *e = getenv(name);
      return e ? atoi(e) : dflt;
    };
    if (const char *e = getenv("MGV_DEAL")) v.deal = !strcmp(e, "tiles") ? 1 : !strcmp(e, "items") ? 2 : !strcmp(e, "pairs") ? 3 : 0;
    v.item = num("MGV_ITEM", 0);
    if (num("MGV_LEAN", 1) == 0) v.kernel = 1;
    if (const char *e = getenv("MGV_XREG")) v.kernel = atoi(e) ? 3 : (v.kernel ? v.kernel : 2);
    v.depth = num("MGV_DEPTH", 0);
    v.dt = num("MGV_DT", 0);
    v.hint_late = num("MGV_HINT_LATE", 0);
    v.hint_cap = (long long)num("MGV_HINT_CAP_KB", 0) * 1024;
    v.prefill = num("MGV_PREFILL", -1);
    v.one_launch = num("MGV_BATCH_SPLIT", 1) == 0;
    v.tensor_fill = num("MGV_TMA", -1);
#endif
    return v;
  }();
  return t;
}

Tuning tuning_for(const mgv_gemv_args &a) {
  Tuning t = env_tuning();
  const int h = a.hints;
  if (h & 3) t.deal = h & 3;
  if (h & MGV_HINT_ITEM_128) t.item = 128;
  if (h & MGV_HINT_ITEM_256) t.item = 256;
  if ((h >> 4) & 3) t.kernel = (h >> 4) & 3;
  if (h & MGV_HINT_ONE_LAUNCH) t.one_launch = 1;
  return t;
}

// warps per block of each kernel: must agree with dispatch_family
int warps_per_block(int variant, int mb) { (void)variant; (void)mb; return 16; }

int count_split_tiles(int U, int ipt, int G) {
  // tiles whose items are owned by more than one block when U items are dealt evenly to G blocks
  const int base = U / G, rem = U % G;
  int n = 0, prev_tile = -1;
  for (int c = 1; c < G; ++c) {
    const int ub = c * base + std::min(c, rem);
    if (ub % ipt != 0 && ub / ipt != prev_tile) {  // a block boundary strictly inside a tile
      ++n;
      prev_tile = ub / ipt;
    }
  }
  return n;
}

mgv_status make_plan_ki(const mgv_gemv_args &a, const DeviceInfo &dev, bool have_ws_hint, Plan &pl, int ki_limit, bool want_lean) {
  const Tuning tune = tuning_for(a);
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
  pl.gshift = group == a.K ? -1 : __builtin_ctz(group);
  pl.two_groups = 0;  // set with the item length below
  pl.has_zero = a.quant_op == MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS;
  if (!a.weights || !a.x || !a.scale || !a.out) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: null weights/x/scale/out");
  if (pl.has_zero && !a.zero) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: FINEGRAINED_SCALE_AND_ZEROS needs zero");
  if (a.flags & ~(MGV_FLAG_OUT_F32_PARTIAL | MGV_FLAG_ACT_RELU | MGV_FLAG_ACT_SILU | MGV_FLAG_PDL | MGV_FLAG_GATED_SILU))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: unknown flag bits 0x%x", a.flags);
  if ((a.flags & MGV_FLAG_ACT_RELU) && (a.flags & MGV_FLAG_ACT_SILU))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: choose one activation");
  const bool gated = (a.flags & MGV_FLAG_GATED_SILU) != 0;
  if (gated && (a.flags & (MGV_FLAG_OUT_F32_PARTIAL | MGV_FLAG_ACT_RELU | MGV_FLAG_ACT_SILU)))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: the gated epilogue excludes fp32 partials and the activation flags");
  if (gated && a.N % 2) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: the gated epilogue pairs rows, N must be even");
  if (a.ldx < a.K || a.ldd < (gated ? a.N / 2 : a.N)) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: ldx < K or ldd < N (N/2 with the gated epilogue)");
  if (a.n_peers < 0 || a.n_peers > MGV_MAX_PEERS)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: n_peers=%d outside 0..%d", a.n_peers, MGV_MAX_PEERS);
  if (a.wait_flag && (!a.wait_state || reinterpret_cast<uintptr_t>(a.wait_flag) % 4 || reinterpret_cast<uintptr_t>(a.wait_state) % 8))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: wait_flag needs a wait_state; 4- and 8-byte aligned");
  if (a.wait_flag && a.wait_sources == 0) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: wait_flag without wait_sources");
  if (a.prefetch && reinterpret_cast<uintptr_t>(a.prefetch) % 16)
    return fail(MGV_STATUS_MISALIGNED, "gemv: the prefetch range must start on a 16-byte boundary");
  for (int q = 0; q < a.n_peers; ++q) {
    if (!a.peer_out[q]) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: peer_out[%d] is null", q);
    if (reinterpret_cast<uintptr_t>(a.peer_out[q]) % ((a.flags & MGV_FLAG_OUT_F32_PARTIAL) ? 4 : 2) ||
        reinterpret_cast<uintptr_t>(a.peer_flag[q]) % 4)
      return fail(MGV_STATUS_MISALIGNED, "gemv: peer_out[%d] / peer_flag[%d] misaligned", q, q);
  }
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
  pl.tile_rows = RG * rpg;
  pl.tiles = (a.N + pl.tile_rows - 1) / pl.tile_rows;
  // Item length: 256 k halves the per-item bookkeeping; it needs groups of at least 128, K a multiple
  // of 128 (its correction table is built per 128 k) and enough items to keep the warps balanced.
  {
    const long long items256 = (long long)pl.tiles * (a.batch_count <= 0 ? 1 : a.batch_count) * ((a.K + 255) / 256);
    const bool long_items = variant == MGV_VARIANT_MMA && group >= 128 && a.K % 128 == 0 && items256 >= (long long)dev.sms * 16 * 6;
    pl.ki = long_items ? 256 : 128;
    if (tune.item == 128) pl.ki = 128;
    if (tune.item == 256 && variant == MGV_VARIANT_MMA && group >= 128 && a.K % 128 == 0) pl.ki = 256;
    pl.ki = std::min(pl.ki, ki_limit);
  }
  pl.two_groups = (group == pl.ki / 2 && a.K > group) ? 1 : 0;
  pl.ipt = (a.K + pl.ki - 1) / pl.ki;
  pl.batch = batch;
  const long long total_tiles = (long long)pl.tiles * batch;
  const long long U = total_tiles * pl.ipt;
  if (U > 0x3fffffff) return fail(MGV_STATUS_UNSUPPORTED, "gemv: more than 2^30 work items (N*K*batch too large)");
  if ((long long)(a.K / group) * a.N > 0x7fffffffLL) return fail(MGV_STATUS_UNSUPPORTED, "gemv: more than 2^31 scales per problem");
  pl.total_tiles = int(total_tiles);
  pl.blocks_per_sm = 1;
  pl.nw = warps_per_block(variant, pl.mb);
  const int NWARP = pl.nw;
  pl.ws_counter_bytes = (size_t(pl.total_tiles) * 4 + 255) / 256 * 256;
  pl.ws_bytes = pl.ws_counter_bytes + size_t(dev.sms) * kMaxBlocksPerSM * 2 * kSlotFloats * 4;

  // ---- how the work is dealt to the blocks ----
  // Equal item ranges cut tiles between blocks; every block then ends with a publish / fence /
  // count / read chain through the scratch, measured at 4 to 6 us on B200.  Whole tiles per block
  // need no scratch but leave blocks idle when the tile count is not a multiple of the grid.
  // Pick the cheaper, with the streaming time estimated at 4 TB/s.
  const int grid_items = int(std::min<long long>(dev.sms, (U + NWARP - 1) / NWARP));
  const int grid_tiles = int(std::min<long long>(dev.sms, total_tiles));
  const double stream_us = double(a.K) * a.N * a.weight_bits / 8 * batch / 4e6;
  const long long tiles_max = (total_tiles + grid_tiles - 1) / grid_tiles;
  const double idle_us = stream_us * (double(tiles_max) * dev.sms / double(total_tiles) - 1.0);
  pl.split_tiles = count_split_tiles(int(U), pl.ipt, grid_items);
  bool split = have_ws_hint && pl.split_tiles > 0 && idle_us > 6.0;
  if (tune.deal == MGV_HINT_DEAL_ITEMS) split = have_ws_hint && pl.split_tiles > 0;
  if (tune.deal == MGV_HINT_DEAL_TILES) split = false;
  pl.align_tiles = split ? 0 : 1;
  // Third way, no scratch: clusters of two blocks own whole tiles and halve their items; the one
  // tile a pair shares is combined through distributed shared memory (about 1 us).  Taken when it
  // shortens the longest block by more than that.
  const int pairs = dev.sms / 2;
  const bool pair_ok = dev.cluster_pairs >= pairs && total_tiles >= pairs && pl.ipt >= 2 && a.M * pl.tile_rows <= 512;
  if (pair_ok && !split) {
    const long long pair_tiles_max = (total_tiles + pairs - 1) / pairs;
    const double tile_us = stream_us / double(total_tiles) * dev.sms;  // one block streaming one tile at full rate
    const double t_tiles = double(tiles_max) * tile_us, t_pairs = double(pair_tiles_max) * tile_us / 2 + 2.5;
    bool use_pairs = t_pairs < t_tiles;
    if (tune.deal == MGV_HINT_DEAL_PAIRS) use_pairs = true;
    if (tune.deal == MGV_HINT_DEAL_TILES) use_pairs = false;
    if (use_pairs) pl.align_tiles = 2;
  }
  if (pl.align_tiles == 2) {
    pl.grid = pairs * 2;
    pl.split_tiles = 0;
    pl.deal_base = int(total_tiles / pairs);
    pl.deal_rem = int(total_tiles % pairs);
  } else if (split) {
    pl.grid = grid_items;
    pl.deal_base = int(U / pl.grid);
    pl.deal_rem = int(U % pl.grid);
  } else {
    pl.grid = grid_tiles;
    pl.split_tiles = 0;
    pl.deal_base = int(total_tiles / pl.grid);
    pl.deal_rem = int(total_tiles % pl.grid);
  }
  long long items_per_block = split ? pl.deal_base + 1 : (long long)(pl.deal_base + (pl.deal_rem ? 1 : 0)) * pl.ipt;
  long long tiles_per_block = split ? (items_per_block + pl.ipt - 1) / pl.ipt + 1 : pl.deal_base + (pl.deal_rem ? 1 : 0);
  if (pl.align_tiles == 2) {
    items_per_block = (items_per_block + 1) / 2;
    tiles_per_block = (tiles_per_block + 1) / 2 + 1;
  }

  // ---- shared memory: partial buffer, correction table, per-warp rings ----
  const int part_slot_bytes = NWARP * a.M * pl.tile_rows * 4;
  pl.slots = int(std::max<long long>(1, std::min<long long>(tiles_per_block, (16 * 1024) / part_slot_bytes)));
  pl.tab_off = (pl.slots * part_slot_bytes + 127) / 128 * 128;
  // x is staged once per block when it is small (it then costs no copy instructions per item);
  // the offset trick of the 4-bit MMA kernels needs the staged, pre-scaled x and its table
  pl.xs_pitch = a.K * 2 + 64;
  const long long xs_bytes = (long long)batch * a.M * pl.xs_pitch;
  const long long tab_bytes = (long long)batch * pl.ipt * 2 * pl.mb * 8;
  const bool stage_x = xs_bytes <= 64 * 1024;
  pl.magic = (variant == MGV_VARIANT_MMA && pl.bits == 4 && stage_x && tab_bytes <= 32 * 1024) ? 1 : 0;
  pl.xs_off = stage_x ? pl.tab_off + (pl.magic ? int((tab_bytes + 127) / 128 * 128) : 0) : -1;
  pl.ring_off = stage_x ? int((pl.xs_off + xs_bytes + 127) / 128 * 128) : pl.tab_off;
  // per-warp prefetch ring: as deep as shared memory allows, no deeper than a warp has items
  const int sb = rpg * 2;
  pl.xstep = stage_x ? 0 : 64 * std::min(a.M, 8);
  const int xr = variant == MGV_VARIANT_MMA ? pl.mb / 8 : 1;
  const int steps = pl.ki / 32;
  const int item_bytes = steps * 512 + 2 * 32 * sb * (pl.has_zero ? 2 : 1) + xr * steps * pl.xstep;
  pl.slot_bytes = item_bytes;
  const long long items_per_warp = (items_per_block + NWARP - 1) / NWARP;
  // the general kernel has 2.1 KB of static shared memory (pair sums, flags) and reads up to 1 KB past its x area
  const int fit = (dev.smem_optin - 4096 - pl.ring_off) / (NWARP * item_bytes);
  if (fit < 1) return fail(MGV_STATUS_UNSUPPORTED, "gemv: shared memory cannot hold one item per warp for this shape");
  pl.depth = int(std::max<long long>(1, std::min<long long>(std::min(fit, MAX_DEPTH), items_per_warp)));
  // + 1 KB: lanes without a batch column read (and ignore) up to 1 KB past their slot's x area
  pl.smem = pl.ring_off + pl.depth * NWARP * item_bytes + 1024;
  // ---- the steady-state kernel (gemv_lean_kernel) where its preconditions hold ----
  pl.lean = 0;
  pl.batch_kernel = 0;
  const int lean_nw = 16;  // 24 and 32 warps were measured slower: their rings are shallower
  // ---- batches of 9..16 rows in one pass over the weights (gemv_batch_kernel), K = 2048 * kpw ----
  if (want_lean && variant == MGV_VARIANT_MMA && pl.mb == 16 && batch == 1 && pl.ki == 128 && a.K % (lean_nw * 128) == 0 &&
      a.K / (lean_nw * 128) <= 4 && a.N % pl.tile_rows == 0 && pl.align_tiles == 1 && a.n_peers == 0 && !a.wait_flag &&
      tune.kernel != 2 && !(group > 2048 && group != a.K)) {
    const int two = group == 64 ? 1 : 0, te = two ? 2 : 1, kpw = a.K / (lean_nw * 128), tg = 2;
    const int slot = 4 * 512 + 32 * sb * te * (pl.has_zero ? 2 : 1);
    const int part_bytes = tg * lean_nw * 2048;  // 2 KB per warp and parked tile whatever M: the slots double as the warp's staging area for x
    const int tab_bytes_b = pl.bits == 4 ? lean_nw * kpw * te * 2 * 128 : 0;
    pl.lean = 1;
    pl.batch_kernel = 1;
    pl.xreg = kpw;
    pl.nw = lean_nw;
    pl.two_groups = two;
    pl.magic = pl.bits == 4 ? 1 : 0;
    pl.slots = tg;
    pl.tab_off = (part_bytes + 127) / 128 * 128;
    pl.xs_off = -1;
    pl.ring_off = pl.tab_off + tab_bytes_b;
    pl.xstep = 0;
    pl.depth = tg;
    pl.slot_bytes = slot;
    pl.smem = pl.ring_off + tg * lean_nw * slot;
    return MGV_STATUS_OK;
  }
  if (want_lean && variant == MGV_VARIANT_MMA && pl.mb == 8 && batch == 1 && pl.ki == 128 && a.K % 128 == 0 &&
      pl.ipt >= lean_nw && a.N % pl.tile_rows == 0 && pl.align_tiles == 1 &&
      (long long)a.N * a.K * a.weight_bits / 8 < (1LL << 32)) {
    const int two = group == 64 ? 1 : 0;
    const int part_tile = lean_nw * a.M * pl.tile_rows * 4;
    const int slots = int(std::max<long long>(1, std::min<long long>(tiles_per_block, (16 * 1024) / part_tile)));
    const int tab_off = (slots * part_tile + 127) / 128 * 128;
    const int tab = pl.bits == 4 ? pl.ipt * (two ? 256 : 128) : 0;
    const int xs_off = tab_off + (tab + 127) / 128 * 128;
    const int ring_off = int((xs_off + (long long)a.M * pl.xs_pitch + 127) / 128 * 128);
    const int slot = 4 * 512 + 32 * sb * (two ? 2 : 1) * (pl.has_zero ? 2 : 1);
    const int lean_fit = (dev.smem_optin - 2048 - ring_off) / (lean_nw * slot);
    // x in registers instead of shared memory (mgv_gemv_tile.cu): K = 16 * 128 * kpw, kpw = 1..4.
    // Measured at least as fast as the staged form for M = 1 and up to 1.7x faster for batches.
    const int kpw = pl.ipt % lean_nw == 0 ? pl.ipt / lean_nw : 0;
    // (a block with a single tile and M = 1 is quicker with x staged: C4 O-proj 4.2 against 4.6 us)
    bool use_xreg = kpw >= 1 && kpw <= 4 && (a.M > 1 || tiles_per_block >= 2);
    if (tune.kernel == 3) use_xreg = kpw >= 1 && kpw <= 4;
    if (tune.kernel == 2) use_xreg = false;
    pl.xreg = 0;
    if (use_xreg) {
      const int te = two ? 2 : 1;
      const int tab_x = pl.bits == 4 ? lean_nw * kpw * te * 128 : 0;
      const int avail = dev.smem_optin - 2048 - tab_x;
      // The ring holds whole tiles: kpw slots per warp and tile.  A shallow ring wins (measured on
      // B200: more requests in flight only queue behind one another): two or three items per warp in
      // flight, i.e. one tile for kpw >= 2, two to four for kpw = 1.
      int dt = kpw == 1 ? (tiles_per_block <= 6 ? 2 : 3) : 1;
      if (kpw == 2 && items_per_warp > 6) dt = 2;
      // in a chain of dependent launches a ring of two tiles with a first fill of one tile wins for K = 4096
      // from two tiles per block on (C2 5.95 -> 5.88 us, QKV 6.31 -> 6.17, C1 4.50 -> 4.45); batches of more than
      // four rows lose with it (C2 M=8: 7.24 against 6.84 us)
      if (kpw == 2 && (a.flags & MGV_FLAG_PDL) && tiles_per_block >= 2 && a.M <= 4) dt = 2;
      if (tune.dt > 0) dt = tune.dt;
      dt = std::max(1, std::min(dt, kpw == 1 ? 4 : (kpw == 2 ? 2 : 1)));
      const int ring_unit = lean_nw * slot;
      long long sl = (avail - dt * kpw * ring_unit) / part_tile;  // room for the partial sums beside the ring
      sl = std::min<long long>(sl, tiles_per_block);
      if (sl >= 1) {
        pl.lean = 1;
        pl.xreg = kpw;
        pl.tile_dt = dt;
        pl.nw = lean_nw;
        pl.two_groups = two;
        pl.magic = pl.bits == 4 ? 1 : 0;
        pl.slots = int(sl);
        pl.tab_off = int((sl * part_tile + 127) / 128 * 128);
        pl.xs_off = -1;
        pl.ring_off = pl.tab_off + tab_x;
        pl.xstep = 0;
        pl.depth = dt * kpw;
        pl.slot_bytes = slot;
        pl.smem = pl.ring_off + pl.depth * ring_unit;
        // A launch that does not overlap its predecessor pays for the issue of its first ring fill (ten
        // copy instructions per lane, 0.5 us of load/store-unit time) on its critical path: there the fill
        // travels as one tiled bulk copy per slot instead (C2 alone: 7.9 -> 7.2 us).  In a chain of
        // dependent launches that time is hidden behind the wait for the predecessor and the copies stay.
        pl.tensor_fill = (!(a.flags & MGV_FLAG_PDL) && !a.wait_flag && a.n_peers == 0) ? 1 : 0;
        if (tune.tensor_fill >= 0) pl.tensor_fill = tune.tensor_fill;
        if (pl.tensor_fill) {
          pl.bar_off = (pl.smem + 127) / 128 * 128;
          pl.smem = pl.bar_off + lean_nw * 8 * 8;  // up to eight 8-byte barriers per warp
        }
        return MGV_STATUS_OK;
      }
    }
    if (lean_fit >= 1) {
      pl.lean = 1;
      pl.nw = lean_nw;
      pl.two_groups = two;
      pl.magic = pl.bits == 4 ? 1 : 0;
      pl.slots = slots;
      pl.tab_off = tab_off;
      pl.xs_off = xs_off;
      pl.ring_off = ring_off;
      pl.xstep = 0;
      pl.depth = std::min(lean_fit, items_per_warp <= 6 ? 2 : 3);  // a shallow ring wins, see the x-in-registers plan above
      if (tune.depth > 0) pl.depth = std::max(1, std::min(lean_fit, tune.depth));
      pl.slot_bytes = slot;
      pl.smem = ring_off + pl.depth * lean_nw * slot;
    }
  }
  return MGV_STATUS_OK;
}

// Long items first; if their slots do not fit shared memory for this shape, short ones.
mgv_status make_plan(const mgv_gemv_args &a, const DeviceInfo &dev, bool have_ws_hint, Plan &pl) {
  const Tuning tune = tuning_for(a);
  if (tune.kernel != 1 && tune.item == 0) {  // (the general kernel on request, and whenever an item length is forced)
    mgv_status st = make_plan_ki(a, dev, have_ws_hint, pl, 128, true);
    if (st == MGV_STATUS_OK && pl.lean) return st;
    pl = Plan{};
  }
  mgv_status st = make_plan_ki(a, dev, have_ws_hint, pl, 256, false);
  if (st == MGV_STATUS_UNSUPPORTED && pl.ki == 256) {
    pl = Plan{};
    st = make_plan_ki(a, dev, have_ws_hint, pl, 128, false);
  }
  return st;
}


template <int BITS, bool HZ, int VAR, int MB, bool MAGIC, bool GENERIC, int KI>
mgv_status launch_one(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  constexpr int NW = 16;
  if (pl.nw != NW) return fail(MGV_STATUS_CUDA_ERROR, "internal: plan and kernel disagree on warps per block");
  return launch_configured<gemv_kernel<BITS, HZ, VAR, MB, NW, MAGIC, GENERIC, KI>>(p, pl, s);
}

template <int BITS, bool HZ, int VAR, int MB, bool MAGIC>
mgv_status launch(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  const bool generic = p.K % pl.ki != 0 || p.two_groups;
  if constexpr (VAR == VAR_MMA) {
    if (pl.ki == 256) {
      if (generic) return launch_one<BITS, HZ, VAR, MB, MAGIC, true, 256>(p, pl, s);
      return launch_one<BITS, HZ, VAR, MB, MAGIC, false, 256>(p, pl, s);
    }
  }
  if (generic) return launch_one<BITS, HZ, VAR, MB, MAGIC, true, 128>(p, pl, s);
  return launch_one<BITS, HZ, VAR, MB, MAGIC, false, 128>(p, pl, s);
}

template <int BITS, bool HZ>
mgv_status dispatch_family(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.variant == MGV_VARIANT_SIMT) {
    if (pl.mb == 1) return launch<BITS, HZ, VAR_SIMT, 1, false>(p, pl, s);
    if (pl.mb == 2) return launch<BITS, HZ, VAR_SIMT, 2, false>(p, pl, s);
    return launch<BITS, HZ, VAR_SIMT, 4, false>(p, pl, s);
  }
  if (pl.lean) return pl.batch_kernel ? launch_batch(p, pl, s) : (pl.xreg ? launch_tile(p, pl, s) : launch_fast(p, pl, s));
  if constexpr (BITS == 4) {
    if (pl.magic) {
      if (pl.mb == 8) return launch<BITS, HZ, VAR_MMA, 8, true>(p, pl, s);
      return launch<BITS, HZ, VAR_MMA, 16, true>(p, pl, s);
    }
  }
  if (pl.mb == 8) return launch<BITS, HZ, VAR_MMA, 8, false>(p, pl, s);
  return launch<BITS, HZ, VAR_MMA, 16, false>(p, pl, s);
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
  // pointers do not matter for sizing: stand-ins where the caller has none yet
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

// ---- a validated, planned call: everything a launch needs, computed once ----------------------
//
// GemvAdaptor::initialize builds Params once and run() only launches
// (gemv/device/gemv_adaptor.h:198-255); mgv_gemv_plan_* is that pair, mgv_gemv does both per call.
struct PreparedPart {
  Plan pl;
  GemvParams p;
};
struct mgv_gemv_plan {
  int parts = 0;  // 1, or 2 for a batch of 9..16 rows served as rows 0..7 and rows 8..M-1
  PreparedPart part[2];
  size_t ws_needed = 0;  // bytes of split-K scratch the first part uses (0: none)
  int device = 0;
};

// The preprocessed weights as a tiled tensor for cp.async.bulk.tensor: bytes, innermost 64 (one
// row group's share of a 32-k step), then the row group (2K bytes apart), then the step along k
// (64 bytes apart).  A box of 64 x 8 x 4 is one item -- 8 row groups x 128 k -- and lands in shared
// memory as [step][row group][64 bytes], the order the kernels read.
static mgv_status encode_weight_map(CUtensorMap *map, const void *w, int N, int K, int bits) {
  using Encode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = nullptr;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!encode) {
      void *fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      MGV_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
      if (q != cudaDriverEntryPointSuccess || !fn) return fail(MGV_STATUS_CUDA_ERROR, "gemv: the driver has no cuTensorMapEncodeTiled");
      encode = reinterpret_cast<Encode>(fn);
    }
  }
  const cuuint64_t group_bytes = cuuint64_t(K) * 2;  // 4 rows of 4-bit or 2 rows of 8-bit weights
  const cuuint64_t dims[3] = {64, cuuint64_t(N) / cuuint64_t(16 / bits), group_bytes / 64};
  const cuuint64_t strides[2] = {group_bytes, 64};
  const cuuint32_t box[3] = {64, 8, 4}, elem[3] = {1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(w), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MGV_STATUS_CUDA_ERROR, "gemv: cuTensorMapEncodeTiled failed (%d)", int(r));
  return MGV_STATUS_OK;
}

static mgv_status prepare_part(const mgv_gemv_args &a, DeviceInfo &dev, PreparedPart &out) {
  Plan &pl = out.pl;
  pl = Plan{};
  const bool have_ws = a.workspace != nullptr;
  mgv_status st = make_plan(a, dev, have_ws, pl);
  if (st != MGV_STATUS_OK) return st;
  if (!pl.align_tiles) {
    if (reinterpret_cast<uintptr_t>(a.workspace) % 256)
      return fail(MGV_STATUS_MISALIGNED, "gemv: workspace must be 256-byte aligned");
    if (a.workspace_bytes < pl.ws_bytes)
      return fail(MGV_STATUS_WORKSPACE_TOO_SMALL, "gemv: workspace has %zu bytes, the shape needs %zu", a.workspace_bytes,
                  pl.ws_bytes);
  }
  GemvParams &p = out.p;
  p = GemvParams{};
  p.w = static_cast<const uint8_t *>(a.weights);
  p.x = static_cast<const __half *>(a.x);
  p.scale = static_cast<const __half *>(a.scale);
  p.zero = pl.has_zero ? static_cast<const __half *>(a.zero) : nullptr;
  p.bias = (a.flags & MGV_FLAG_OUT_F32_PARTIAL) ? nullptr : static_cast<const __half *>(a.bias);
  p.out = a.out;
  p.ws_counters = static_cast<int *>(a.workspace);
  p.ws_slots = a.workspace ? reinterpret_cast<float *>(static_cast<uint8_t *>(a.workspace) + pl.ws_counter_bytes) : nullptr;
  p.ldx = a.ldx; p.ldd = a.ldd;
  p.bs_w = a.batch_stride_weights; p.bs_x = a.batch_stride_x; p.bs_scale = a.batch_stride_scale;
  p.bs_bias = a.batch_stride_bias; p.bs_out = a.batch_stride_out;
  p.alpha = a.alpha; p.beta = a.beta;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.gshift = pl.gshift; p.two_groups = pl.two_groups; p.ki = pl.ki;
  p.tiles = pl.tiles; p.ipt = pl.ipt; p.total_tiles = pl.total_tiles;
  p.align_tiles = pl.align_tiles; p.slots = pl.slots; p.depth = pl.depth; p.ring_off = pl.ring_off; p.slot_bytes = pl.slot_bytes;
  p.xstep = pl.xstep; p.xs_off = pl.xs_off; p.xs_pitch = pl.xs_pitch;
  p.tab_off = pl.tab_off; p.deal_base = pl.deal_base; p.deal_rem = pl.deal_rem; p.batch = pl.batch; p.flags = a.flags;
  p.wait_flag = static_cast<const unsigned *>(a.wait_flag);
  p.wait_state = static_cast<unsigned long long *>(a.wait_state);
  p.wait_delta = a.wait_delta;
  p.wait_sources = a.wait_sources;
  p.err_word = dev.err_word;
  p.prefetch = static_cast<const uint8_t *>(a.prefetch);
  p.prefetch_bytes = a.prefetch ? a.prefetch_bytes : 0;
  p.n_peers = a.n_peers;
  for (int q = 0; q < a.n_peers; ++q) {
    p.peer_out[q] = a.peer_out[q];
    p.peer_flag[q] = static_cast<unsigned *>(a.peer_flag[q]);
  }
  // ring slots filled before the wait for the previous kernel: measured best on B200 -- 4-bit: 3 (C2 7.2 / 6.8 / 7.3 /
  // 7.5 us at 2 / 3 / 4 / 5); 8-bit: 2 (C1 5.16 against 5.30 us at 3)
  p.prefill = pl.bits == 8 ? 2 : 3;
  const Tuning tune = tuning_for(a);
  // with the bulk fill x is asked for behind one slot only and the rest of the ring follows it (measured best on
  // every shape but the two-tile ring of K = 4096, which wants three)
  if (pl.tensor_fill) p.prefill = (pl.xreg == 2 && pl.tile_dt == 2) ? 3 : 1;
  else if (pl.lean && pl.xreg == 2 && pl.tile_dt == 2 && !pl.batch_kernel) p.prefill = 2;
  if (tune.prefill >= 0) p.prefill = tune.prefill;
  p.hint_late = tune.hint_late;
  // (a driver that refuses the map costs the bulk fill, not the call: the per-lane copies serve)
  if (pl.tensor_fill && encode_weight_map(&p.w_map, a.weights, a.N, a.K, a.weight_bits) != MGV_STATUS_OK) pl.tensor_fill = 0;
  p.bar_off = pl.tensor_fill ? pl.bar_off : 0;
  if (tune.hint_cap > 0 && p.prefetch_bytes > size_t(tune.hint_cap)) p.prefetch_bytes = size_t(tune.hint_cap);
  return MGV_STATUS_OK;
}

// Batches of 9..16 rows whose first eight rows would run on a steady-state kernel are served as
// two launches (rows 0..7, rows 8..M-1): twice the weight traffic, but both passes at the
// steady-state kernels' rate, and the second finds part of the weights in L2 -- measured faster
// than the one general-kernel launch with x travelling in the ring (C3 M=16).  Not with peers or
// waits (their counts are per launch) or batched problems.
static mgv_status prepare(const mgv_gemv_args *a, mgv_gemv_plan &out) {
  if (!a) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv: null args");
  mgv_status st = MGV_STATUS_OK;
  DeviceInfo *dev = device_info(&st);
  if (!dev) return st;
  MGV_CUDA_TRY(cudaGetDevice(&out.device));
  out.parts = 1;
  if ((st = prepare_part(*a, *dev, out.part[0])) != MGV_STATUS_OK) return st;
  const bool may_split = !out.part[0].pl.batch_kernel && a->M > 8 && a->M <= 16 && !a->n_peers && !a->wait_flag && a->batch_count <= 1 &&
                         a->variant != MGV_VARIANT_SIMT && !tuning_for(*a).one_launch;
  if (may_split) {
    const size_t esz = (a->flags & MGV_FLAG_OUT_F32_PARTIAL) ? 4 : 2;
    mgv_gemv_args lo = *a, hi = *a;
    lo.M = 8;
    hi.M = a->M - 8;
    hi.x = static_cast<const char *>(a->x) + size_t(8) * a->ldx * 2;
    hi.out = static_cast<char *>(a->out) + size_t(8) * a->ldd * esz;
    PreparedPart first;
    if (prepare_part(lo, *dev, first) == MGV_STATUS_OK && first.pl.lean) {
      out.part[0] = first;
      if ((st = prepare_part(hi, *dev, out.part[1])) != MGV_STATUS_OK) return st;
      out.parts = 2;
    }
  }
  out.ws_needed = out.part[0].pl.split_tiles ? out.part[0].pl.ws_bytes : 0;
  return MGV_STATUS_OK;
}

static mgv_status launch_part(const PreparedPart &pp, cudaStream_t s) {
  const Plan &pl = pp.pl;
  if (pl.bits == 4) return pl.has_zero ? dispatch_family<4, true>(pp.p, pl, s) : dispatch_family<4, false>(pp.p, pl, s);
  return pl.has_zero ? dispatch_family<8, true>(pp.p, pl, s) : dispatch_family<8, false>(pp.p, pl, s);
}

static mgv_status launch_prepared(const mgv_gemv_plan &pr, cudaStream_t s) {
  for (int i = 0; i < pr.parts; ++i) {
    mgv_status st = launch_part(pr.part[i], s);
    if (st != MGV_STATUS_OK) return st;
  }
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_gemv_launch_info(const mgv_gemv_args *a, mgv_launch_info *info) {
  if (!info) return fail(MGV_STATUS_INVALID_ARGUMENT, "launch_info: null info");
  mgv_gemv_plan pr;
  mgv_status st = prepare(a, pr);
  if (st != MGV_STATUS_OK) return st;
  const Plan &pl = pr.part[0].pl;  // two launches: the first one's geometry is reported
  info->variant = pl.variant;
  info->grid = pl.grid;
  info->block = pl.nw * 32;
  info->stages = pl.depth;
  info->smem_bytes = pl.smem;
  info->tile_rows = pl.tile_rows;
  info->k_slice = pl.ki;
  info->split_tiles = pl.split_tiles;
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_gemv(const mgv_gemv_args *a, mgv_stream_t s) {
  mgv_gemv_plan pr;
  mgv_status st = prepare(a, pr);
  if (st != MGV_STATUS_OK) return st;
  return launch_prepared(pr, s);
}

extern "C" mgv_status mgv_gemv_plan_create(const mgv_gemv_args *a, mgv_gemv_plan **plan) {
  if (!plan) return fail(MGV_STATUS_INVALID_ARGUMENT, "plan_create: null plan pointer");
  *plan = nullptr;
  mgv_gemv_plan *pr = new (std::nothrow) mgv_gemv_plan;
  if (!pr) return fail(MGV_STATUS_CUDA_ERROR, "plan_create: out of host memory");
  mgv_status st = prepare(a, *pr);
  if (st != MGV_STATUS_OK) {
    delete pr;
    return st;
  }
  *plan = pr;
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_gemv_plan_run(const mgv_gemv_plan *plan, mgv_stream_t s) {
  if (!plan) return fail(MGV_STATUS_INVALID_ARGUMENT, "plan_run: null plan");
  int dev = 0;
  MGV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev != plan->device) return fail(MGV_STATUS_INVALID_ARGUMENT, "plan_run: the plan was made on device %d, current is %d", plan->device, dev);
  return launch_prepared(*plan, s);
}

extern "C" void mgv_gemv_plan_destroy(mgv_gemv_plan *plan) { delete plan; }

// ---- mgv_gemv for callers that may not allocate device memory ----------------------------------
//
// Some callers of a GEMV cannot hand over scratch of their own: code running while a stream is
// being captured (cudaMalloc is not allowed there), an inference-runtime plug-in whose enqueue hook
// gets a fixed memory budget, a real-time loop that must not touch the allocator, a host language
// binding that has no device allocator at hand.  For them the split-K scratch lives in the
// library image itself: a file-scope device array of kStaticScratchBytes that every GPU loading the
// library holds until the process exits.
constexpr size_t kStaticScratchBytes = size_t(4) << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` only names the symbol; the kernel needs the array's address ON
// THE CURRENT DEVICE, looked up once per device.
static mgv_status static_scratch_address(void **ptr) {
  static void *addr[64];
  static std::mutex mu;
  int dev = 0;
  MGV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MGV_STATUS_UNSUPPORTED, "gemv_static_scratch: device index %d beyond 63", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void *p = nullptr;
    MGV_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    addr[dev] = p;
  }
  *ptr = addr[dev];
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_gemv_static_scratch(const mgv_gemv_args *a, mgv_stream_t s) {
  if (!a) return fail(MGV_STATUS_INVALID_ARGUMENT, "gemv_static_scratch: null args");
  // plan once as if the caller had scratch: the plan says whether and how much of it is used
  mgv_gemv_args b = *a;
  void *scratch = nullptr;
  mgv_status st = static_scratch_address(&scratch);
  if (st != MGV_STATUS_OK) return st;
  b.workspace = scratch;
  b.workspace_bytes = size_t(1) << 62;  // sizing only; the real bound is checked right below
  mgv_gemv_plan pr;
  if ((st = prepare(&b, pr)) != MGV_STATUS_OK) return st;
  if (pr.ws_needed > kStaticScratchBytes)
    return fail(MGV_STATUS_WORKSPACE_TOO_SMALL,
                "gemv_static_scratch: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu; "
                "use mgv_gemv with caller-owned scratch",
                pr.ws_needed, kStaticScratchBytes);
  if (pr.ws_needed) {
    // The array keeps whatever the previous call left.  Only the per-tile arrival counters at its
    // start must read zero when a launch begins; the slots behind them are written before they are read.
    MGV_CUDA_TRY(cudaMemsetAsync(scratch, 0, pr.part[0].pl.ws_counter_bytes, s));
  }
  return launch_prepared(pr, s);
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


