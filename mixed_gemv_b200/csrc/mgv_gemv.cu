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
// Three kernels share this scheme:
//   * gemv_kernel       everything: both families, M <= 16, ragged N and K, groups of 64, batched
//                       problems, all three ways of dealing the work;
//   * gemv_lean_kernel  the MMA family's common decode shapes with the per-item bookkeeping cut
//                       down (the general kernel was issue-bound on it), x staged in shared memory;
//   * gemv_xreg_kernel  the same for K = 4096 and 8192 with each warp's x fragments in registers:
//                       no staged x, no block barrier before the arithmetic -- the bench kernel.
// The host (make_plan) picks by shape; the epilogue (store_out), the exchange (signal_peers,
// wait_enter / wait_arrived) and the dependent-launch handling are common to all three.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "mgv_common.cuh"

namespace mgv {

// An item is KI = 128 or 256 consecutive k of a row tile (a kernel template parameter): 256 halves
// the per-item bookkeeping for shapes with enough items, 128 keeps small calls balanced.
constexpr int RG = 8;                   // row groups per tile
constexpr int MAX_DEPTH = 8;            // deepest per-warp prefetch ring
constexpr int VAR_SIMT = 1, VAR_MMA = 2;
constexpr int kSlotFloats = 16 * 32;    // largest batch bucket x largest tile: one scratch slot size for all kernels
constexpr int kMaxBlocksPerSM = 4;      // scratch is sized for this many resident blocks per SM

// Phase timestamps for kernel tuning; compiled in only with -DMGV_TRACE (never in the library).
// Four launches are kept apart by bits 12-13 of their output address.
#ifdef MGV_TRACE
__device__ unsigned long long g_trace[8 * 1024];
#define MGV_TRACE_MARK(k)                                                                  \
  do {                                                                                     \
    if (threadIdx.x == 0 && blockIdx.x < 256)                                              \
      g_trace[(((reinterpret_cast<uintptr_t>(p.out) >> 12) & 3) * 256 + blockIdx.x) * 8 + (k)] = global_timer_ns(); \
  } while (0)
#else
#define MGV_TRACE_MARK(k) do { } while (0)
#endif

// Set by a kernel whose bounded wait gave up; read and cleared by mgv_device_error_state.
__device__ int g_device_error_word;

struct GemvParams {
  const uint8_t *w;
  const __half *x;
  const __half *scale;
  const __half *zero;
  const __half *bias;
  void *out;
  float *ws_slots;   // [grid][2][kSlotFloats] partial sums of split tiles
  int *ws_counters;  // [batch*tiles] arrivals per split tile (zero between launches)
  int64_t ldx, ldd;
  int64_t bs_w, bs_x, bs_scale, bs_bias, bs_out;
  float alpha, beta;
  int M, N, K;
  int gshift;        // log2(group_size) for power-of-two groups, -1 when the one group spans K
  int two_groups;    // group_size == 64: an item spans two groups
  int tiles;         // row tiles per problem
  int ipt;           // items per tile = ceil(K / KI)
  int ki;            // KI of the launched kernel
  int total_tiles;   // batch_count * tiles
  int align_tiles;   // 1: blocks own whole tiles (no scratch); 0: blocks own equal item ranges;
                     // 2: PAIRS of blocks (a cluster of two) own whole tiles and halve their items
  int slots;         // tile slots of the shared-memory partial buffer (tiles per round)
  int depth;         // items each warp keeps in flight (slots of its shared-memory ring)
  int ring_off;      // byte offset of the rings in dynamic shared memory
  int slot_bytes;    // bytes of one ring slot
  int tab_off;       // byte offset of the per-item correction table (MAGIC kernels)
  int deal_base, deal_rem;  // items (or tiles, align_tiles) per block: the first deal_rem blocks get one more
  int batch;         // batch_count
  int prefill;       // ring slots filled before the block-wide set-up (the rest follow its barrier)
  int xstep;         // bytes of x one step of one slot holds per 8 batch columns: 64 * min(M, 8); 0 when x is staged
  int xs_off;        // byte offset of the block's staged copy of x in shared memory, -1 when x travels in the ring
  int xs_pitch;      // bytes between staged rows of x: 2K + 64 (the 64 spreads the rows over the banks)
  int flags;
  int n_peers;       // destinations of the fused output exchange (0: none)
  void *peer_out[MGV_MAX_PEERS];        // other GPUs' output buffers, laid out like out (fp16, or fp32 partials)
  unsigned *peer_flag[MGV_MAX_PEERS];   // their arrival counters (entries may be null)
  const unsigned *wait_flag;            // this GPU's arrival counter the kernel waits on before it reads x (or null)
  unsigned long long *wait_state;       // launches that used this wait so far
  unsigned wait_delta;                  // arrivals one earlier launch of the chain brings
};

template <int BITS>
struct Geometry {
  static constexpr int RPG = 16 / BITS;  // rows per 16-byte unit
  static constexpr int TILE_ROWS = RG * RPG;
};

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

__device__ __forceinline__ uint32_t dup_lo(uint32_t v) { return __byte_perm(v, v, 0x1010); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t v) { return __byte_perm(v, v, 0x3232); }
__device__ __forceinline__ float half_lo(uint32_t v) { return __half2float(__ushort_as_half(uint16_t(v & 0xffffu))); }
__device__ __forceinline__ float half_hi(uint32_t v) { return __half2float(__ushort_as_half(uint16_t(v >> 16))); }

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

__device__ __forceinline__ void cp_async_cg16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most n of this thread's most recent groups are still pending (n < MAX_DEPTH)
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}

__device__ __forceinline__ float apply_act(float v, int flags) {
  if (flags & MGV_FLAG_ACT_RELU) v = fmaxf(v, 0.0f);
  if (flags & MGV_FLAG_ACT_SILU) v = v / (1.0f + __expf(-v));
  return v;
}

// shared-memory accesses by 32-bit shared address with a compile-time byte offset
template <int OFF>
__device__ __forceinline__ uint4 lds128_at(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32_at(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ void cp16_at(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0+%1], [%2], 16;" ::"r"(dst), "n"(OFF), "l"(src) : "memory");
}
// the copy happens only where `on` is set; a predicate instead of a branch keeps the warp converged
__device__ __forceinline__ void cp16_if(uint32_t dst, const void *src, bool on) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0], [%1], 16;\n\t}" ::"r"(dst), "l"(src),
               "r"(int(on))
               : "memory");
}
template <int BYTES, int OFF>
__device__ __forceinline__ void cp_small_at(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0+%1], [%2], %3;" ::"r"(dst), "n"(OFF), "l"(src), "n"(BYTES) : "memory");
}

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

// One 16-byte unit -> hh[row][pair] = half2 of the signed integer weights (k, k+1), unscaled.
template <int BITS>
__device__ __forceinline__ void convert_unit(const uint4 wv, uint32_t (&hh)[16 / BITS][4]) {
  const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
  if constexpr (BITS == 4) {
#pragma unroll
    for (int r = 0; r < 4; ++r) cvt_u4x8(wr[r], hh[r]);
  } else {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      uint32_t lo[2], hi[2];
      cvt_u8x4(wr[2 * r], lo);
      cvt_u8x4(wr[2 * r + 1], hi);
      hh[r][0] = lo[0]; hh[r][1] = lo[1]; hh[r][2] = hi[0]; hh[r][3] = hi[1];
    }
  }
}

// 4-bit unit -> hh[row][pair] WITHOUT the offset fix-up: pairs 0 and 2 hold 1024 + u, pairs 1
// and 3 hold 1024 + 16u (u = weight + 8).  The caller multiplies pairs 1 and 3 by x/16 and
// removes 1032*x resp. 72*x through a precomputed per-item correction.
__device__ __forceinline__ void convert_unit_raw(const uint4 wv, uint32_t (&hh)[4][4]) {
  const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint32_t top = wr[r] >> 8;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(hh[r][0]) : "r"(wr[r]));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(hh[r][1]) : "r"(wr[r]));
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(hh[r][2]) : "r"(top));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(hh[r][3]) : "r"(top));
  }
}

// The lane's scales (or zeros) of one group as packed half2 words: RPG/2 words.
template <int BITS, int OFF>
__device__ __forceinline__ void load_rows(uint32_t addr, uint32_t (&v)[16 / BITS / 2]) {
  v[0] = lds32_at<OFF>(addr);
  if constexpr (BITS == 4) v[1] = lds32_at<OFF + 4>(addr);
}

template <int N>
__device__ __forceinline__ void dup_rows(const uint32_t (&v)[N], uint32_t (&d)[2 * N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) { d[2 * i] = dup_lo(v[i]); d[2 * i + 1] = dup_hi(v[i]); }
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

// ---- a warp leaves a tile: park its partial sums in dst[m][row] and clear the accumulators ----
template <int BITS, int VAR, int MB, int NACC>
__device__ __forceinline__ void flush_acc(float *dst, float (&acc)[NACC], int M, int g, int t) {
  constexpr int RPG = Geometry<BITS>::RPG, TILE_ROWS = Geometry<BITS>::TILE_ROWS;
  if constexpr (VAR == VAR_MMA) {
#pragma unroll
    for (int c8 = 0; c8 < MB / 8; ++c8)
#pragma unroll
      for (int q = 0; q < RPG / 2; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = c8 * 8 + 2 * t + (e & 1);
          const int row = g * RPG + 2 * q + (e >> 1);
          if (col < M) dst[col * TILE_ROWS + row] = acc[(c8 * (RPG / 2) + q) * 4 + e];
        }
  } else {
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
      for (int r = 0; r < RPG; ++r) {
        float v = acc[(m * RPG + r) * 2] + acc[(m * RPG + r) * 2 + 1];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (t == 0 && m < M) dst[m * TILE_ROWS + g * RPG + r] = v;
      }
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
}

// Programmatic dependent launch.  launch_dependents lets the next kernel of the stream start its
// blocks as soon as SMs free up; wait holds this kernel until the previous one has completed and
// its writes are visible.  Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// thread-block-cluster helpers (pairs of blocks that halve a tile range between them)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// reads a float from the same shared-memory address in the block of the given rank of the cluster
__device__ __forceinline__ float ld_peer_shared(const float *own_addr, int rank) {
  uint32_t peer;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(smem_u32(own_addr)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer) : "memory");
  return v;
}

// Consumer side of the exchange.  wait_enter: called by thread 0 at kernel entry, BEFORE the
// block lets dependent launches start, so that the counts of this launch all precede those of
// the next (a dependent grid starts only after every block of this one has passed that point);
// returns the arrivals this launch must see: (launches before it) * delta.
__device__ __forceinline__ unsigned wait_enter(const GemvParams &p) {
  const unsigned long long my = atomicAdd(p.wait_state, 1ull);
  return unsigned((my / gridDim.x) * p.wait_delta);
}
// wait_arrived: thread 0 polls the counter (bounded, about a second), then the block meets.
__device__ __forceinline__ void wait_arrived(const GemvParams &p, unsigned target) {
  if (threadIdx.x == 0) {
    const uint64_t t0 = global_timer_ns();
    for (bool done = false; !done;) {
      for (int i = 0; i < 64 && !done; ++i) {
        unsigned v;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_flag) : "memory");
        done = int(v - target) >= 0;
      }
      if (!done && global_timer_ns() - t0 > 1000000000ull) {
        atomicOr(&g_device_error_word, 0x40);
        done = true;
      }
    }
    asm volatile("fence.acquire.sys;" ::: "memory");  // what the counted blocks stored is visible from here on
  }
  __syncthreads();
}

// First item of block c when the items (or tiles) are dealt as evenly as integers allow:
// the first `rem` blocks get base+1.
__device__ __forceinline__ int range_lo(int c, int base, int rem) { return c * base + min(c, rem); }
__device__ __forceinline__ int range_owner(int u, int base, int rem) {
  const int cut = rem * (base + 1);
  return u < cut ? u / (base + 1) : rem + (u - cut) / base;
}

// out = half(act(alpha*acc + beta*bias)) or the fp32 partial (gemv_adaptor's LinearCombination
// epilogue, epilogue/threadblock/epilogue.h:78-97)
template <int TILE_ROWS>
__device__ __forceinline__ void store_out(const GemvParams &p, int tg, int i, float v) {
  const int b = p.total_tiles == p.tiles ? 0 : tg / p.tiles, tile = tg - b * p.tiles;
  const int m = i / TILE_ROWS, n = tile * TILE_ROWS + i % TILE_ROWS;
  if (n >= p.N) return;
  if (p.flags & MGV_FLAG_GATED_SILU) {
    // rows n (even: gate) and n + 1 (up) sit in neighbouring lanes: N is even, so both or neither are here
    float r = p.alpha * v;
    if (p.bias) r += p.beta * __half2float(p.bias[size_t(b) * p.bs_bias + n]);
    const float other = __shfl_xor_sync(__activemask(), r, 1);
    if ((n & 1) == 0) {
      const size_t og = size_t(b) * p.bs_out + size_t(m) * p.ldd + (n >> 1);
      const __half h = __float2half_rn(r / (1.0f + __expf(-r)) * other);
      static_cast<__half *>(p.out)[og] = h;
      for (int q = 0; q < p.n_peers; ++q) static_cast<__half *>(p.peer_out[q])[og] = h;
    }
    return;
  }
  const size_t o = size_t(b) * p.bs_out + size_t(m) * p.ldd + n;
  if (p.flags & MGV_FLAG_OUT_F32_PARTIAL) {
    const float r = p.alpha * v;
    static_cast<float *>(p.out)[o] = r;
    for (int q = 0; q < p.n_peers; ++q) static_cast<float *>(p.peer_out[q])[o] = r;  // K-split: partials to every GPU
  } else {
    float r = p.alpha * v;
    if (p.bias) r += p.beta * __half2float(p.bias[size_t(b) * p.bs_bias + n]);
    const __half h = __float2half_rn(apply_act(r, p.flags));
    static_cast<__half *>(p.out)[o] = h;
    for (int q = 0; q < p.n_peers; ++q) static_cast<__half *>(p.peer_out[q])[o] = h;  // peer stores: the exchange of an N-split layer
  }
}

// Fused output exchange: called by every thread of a block after the block's last output
// store.  The barrier orders all threads' stores before the fence of the signalling threads;
// fence + release make them visible system-wide before the peer sees the count.
__device__ __forceinline__ void signal_peers(const GemvParams &p) {
  if (p.n_peers == 0) return;
  __syncthreads();
  if (int(threadIdx.x) < p.n_peers) {
    unsigned *flag = p.peer_flag[threadIdx.x];
    // release at system scope: the block's stores (ordered before this thread by the barrier)
    // are visible to the peer before the count is
    if (flag) asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
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
  if (i_begin >= i_end) {
    signal_peers(p);
    return;
  }
  MGV_TRACE_MARK(0);
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
    MGV_TRACE_MARK(7);
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
    MGV_TRACE_MARK(1);
    for (int d = prefill; d < D; ++d) {  // one group per slot, empty groups keep the count uniform
      if (n_issue > 0) issue(ring + d * slot_bytes);
      cp_async_commit();
    }

    {
      int cur_tile = -1;
      uint32_t slot = ring;
      bool first = true;
      while (n_compute > 0) {
        cp_async_wait_pending(D - 1);  // the oldest group, i.e. this item, has landed
        if (first) { MGV_TRACE_MARK(2); first = false; }
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
      MGV_TRACE_MARK(3);
      if (cur_tile >= 0)
        flush_acc<BITS, VAR, MB>(part + size_t(cur_tile - ta) * slot_floats + warp * M * TILE_ROWS, acc, M, g, t);
    }
    __syncthreads();
    MGV_TRACE_MARK(4);

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
      MGV_TRACE_MARK(5);
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
    MGV_TRACE_MARK(6);
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
template <int I, int N, class F>
__device__ __forceinline__ void static_for(F &&f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}

template <int OFF>
__device__ __forceinline__ uint2 lds64_at(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}

template <int N>
__device__ __forceinline__ void cp_async_wait_fixed() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

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
    signal_peers(p);
    return;
  }
  MGV_TRACE_MARK(0);

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
      if (p.wait_flag) count_in();
      pdl_wait();
      if (p.wait_flag) wait_arrived(p, sh_wait_target);  // the peers' slices this call consumes have landed
      MGV_TRACE_MARK(7);
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
      MGV_TRACE_MARK(5);
      __syncthreads();
      MGV_TRACE_MARK(1);
      first_round = false;
    }
    for (; filled < D; ++filled) issue(ring + filled * SLOT, filled < n);

    uint32_t slot = ring;
    for (int j = 0; j < n; ++j) {
      cp_async_wait_fixed<D - 1>();  // the oldest group, i.e. this item, has landed
#ifdef MGV_TRACE
      if (j == 0 && ta == t_first) MGV_TRACE_MARK(2);
#endif
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
    MGV_TRACE_MARK(3);
    if (c_tile < tb - ta) flush_acc<BITS, VAR_MMA, 8>(part + size_t(c_tile) * slot_floats + warp * n_out, acc, M, g, t);
    __syncthreads();
    MGV_TRACE_MARK(4);
    // every warp has visited every tile of the round (ipt >= NW): add the warps' sums in warp order
    for (int e = threadIdx.x; e < (tb - ta) * n_out; e += THREADS) {
      const int tile = e / n_out, i = e - tile * n_out;
      const float *src = part + size_t(tile) * slot_floats + i;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < NW; ++w) v += src[w * n_out];
      store_out<TILE_ROWS>(p, ta + tile, i, v);
    }
    if (tb < t_end) __syncthreads();  // part is reused by the next round
    MGV_TRACE_MARK(6);
  }
  signal_peers(p);
}

// Arithmetic of one item with the x fragments in registers (see gemv_xreg_kernel): as
// lean_compute4, xv[st] being the lane's x chunk of step st (hi pairs already scaled by 1/16).
template <bool HAS_ZERO, bool TWO>
__device__ __forceinline__ void xreg_compute4(uint32_t wa, uint32_t sa, uint32_t tab, const uint4 (&xv)[4], float (&acc)[8]) {
  constexpr int SB = 8, ZO = (TWO ? 64 : 32) * SB;
  static_for<0, TWO ? 2 : 1>([&](auto h_c) {
    constexpr int H = decltype(h_c)::value;
    constexpr int ST0 = TWO ? 2 * H : 0, ST1 = TWO ? 2 * H + 2 : 4;
    const uint4 i0 = lds128_at<H * 128>(tab), i1 = lds128_at<H * 128>(tab);
    float ci[2][4] = {{__uint_as_float(i0.x), __uint_as_float(i0.y), __uint_as_float(i0.z), __uint_as_float(i0.w)},
                      {__uint_as_float(i1.x), __uint_as_float(i1.y), __uint_as_float(i1.z), __uint_as_float(i1.w)}};
    static_for<ST0, ST1>([&](auto st_c) {
      constexpr int ST = decltype(st_c)::value;
      const uint4 wv = lds128_at<ST * 512>(wa);
      uint32_t hh[4][4];
      convert_unit_raw(wv, hh);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        mma_16816(ci[q], hh[2 * q][0], hh[2 * q + 1][0], hh[2 * q][1], hh[2 * q + 1][1], xv[ST].x, xv[ST].y);
        mma_16816(ci[q], hh[2 * q][2], hh[2 * q + 1][2], hh[2 * q][3], hh[2 * q + 1][3], xv[ST].z, xv[ST].w);
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

// The same for 8-bit weights (scaled in fp16 with the reference's rounding points, see lean_compute8).
template <bool HAS_ZERO, bool TWO>
__device__ __forceinline__ void xreg_compute8(uint32_t wa, uint32_t sa, const uint4 (&xv)[4], float (&acc)[4]) {
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
      uint32_t hh[2][4];
      convert_unit<8>(wv, hh);
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hh[r][i] = hmul2_rn(hh[r][i], s2[r]);
          if constexpr (HAS_ZERO) hh[r][i] = hadd2_rn(hh[r][i], z2[r]);
        }
      mma_16816(acc, hh[0][0], hh[1][0], hh[0][1], hh[1][1], xv[ST].x, xv[ST].y);
      mma_16816(acc, hh[0][2], hh[1][2], hh[0][3], hh[1][3], xv[ST].z, xv[ST].w);
    });
  });
}

// The steady-state kernel with x in REGISTERS, M <= 8, K = KPW * 16 * 128 (KPW = 2
// or 4: K = 4096 or 8192).  With sixteen warps taking a tile's items round-robin, warp w only ever
// meets the k ranges w, w+16, ... of every tile: its x fragments for those KPW ranges (16 registers
// each) are loaded once, straight from global memory, and stay in registers.  Shared memory then
// holds no x at all -- which is what lets batches of 5..8 rows keep a deep ring at K = 8192, where
// the staged copy of x alone would take 131 KB -- there is no block-wide staging barrier, and an
// item costs four shared-memory loads less.  The correction table of the 4-bit kernels is per warp
// (built with shuffles from the registers): [KPW][groups per item][4 lane quarters] entries of 32 bytes.
template <int BITS, bool HAS_ZERO, bool TWO, int D, int KPW>
__global__ void __launch_bounds__(512, 1) gemv_xreg_kernel(const __grid_constant__ GemvParams p) {
  constexpr int NW = 16, THREADS = 512, KI = 128, STEPS = 4, TE = TWO ? 2 : 1;
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
  auto count_in = [&]() {  // see gemv_lean_kernel
    if (threadIdx.x == 0) sh_wait_target = wait_enter(p);
    __syncthreads();
    pdl_launch_dependents();
  };
  if (!p.wait_flag) pdl_launch_dependents();
  if (t_first >= t_end) {
    if (p.wait_flag) count_in();
    signal_peers(p);
    return;
  }
  MGV_TRACE_MARK(0);

  const uint32_t group_bytes = uint32_t(p.K) * 2, tile_bytes = group_bytes * RG;
  const uint8_t *wl = p.w + size_t(g) * group_bytes + t * 16 + uint32_t(warp) * (KI * 2);
  const __half *sl = p.scale + g * RPG;
  const __half *zl = HAS_ZERO ? p.zero + g * RPG : nullptr;
  const int gs = p.gshift < 0 ? 31 : p.gshift - 7;
  const uint32_t n_cols = uint32_t(p.N);
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t ring = smem_base + p.ring_off + uint32_t(warp) * (D * SLOT);
  const uint32_t ring_end = ring + D * SLOT;
  const uint32_t w_lane = lane * 16, s_lane = STEPS * 512 + lane * SB;
  const uint32_t tab_warp = smem_base + p.tab_off + uint32_t(warp) * (KPW * TE * 128);
  const uint32_t tab_lane = tab_warp + t * 32;
  const int n_out = M * TILE_ROWS, slot_floats = NW * n_out;

  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
  uint4 xr[KPW][4];
  bool first_round = true;

  for (int ta = t_first; ta < t_end; ta += p.slots) {
    const int tb = min(t_end, ta + p.slots);
    const int ntl = tb - ta, n = ntl * KPW;  // this warp's items: KPW per tile, k ranges warp + 16 j
    int i_tg = ta, i_j = 0;                  // the next item to copy
    auto issue = [&](uint32_t slot, bool on) {
      const uint32_t ki = uint32_t(warp) + uint32_t(i_j) * NW;
      const uint32_t woff = uint32_t(i_tg) * tile_bytes + uint32_t(i_j) * (NW * KI * 2);
      const uint32_t grp = TWO ? ki * 2 : (ki >> gs);
      const uint32_t soff = grp * n_cols + uint32_t(i_tg) * TILE_ROWS;
      lean_copy_item<SB, HAS_ZERO, TWO>(slot + w_lane, wl + woff, slot + s_lane, sl + soff, zl + soff, n_cols, on);
      if (++i_j == KPW) { i_j = 0; ++i_tg; }
    };
    int filled = 0;
    if (first_round) {
      const int pf = min(D, p.prefill);
      for (; filled < pf; ++filled) issue(ring + filled * SLOT, filled < n);
      if (p.wait_flag) count_in();
      pdl_wait();
      if (p.wait_flag) wait_arrived(p, sh_wait_target);
      MGV_TRACE_MARK(7);
      // the lane's x: batch row g (lanes without a row read row M-1 and are ignored), chunk t of every step
      const __half *xl = p.x + size_t(min(g, M - 1)) * p.ldx + warp * KI + t * 8;
#pragma unroll
      for (int j = 0; j < KPW; ++j)
#pragma unroll
        for (int st = 0; st < STEPS; ++st) xr[j][st] = __ldcg(reinterpret_cast<const uint4 *>(xl + j * (NW * KI) + st * 32));
      // Per-warp correction table, by the tensor cores: an A fragment holding -1032 on the k
      // positions of the lo pairs and -72 on those of the hi pairs turns the x fragments into
      // -(1032*sum lo + 72*sum hi) per batch column -- already in the accumulator layout
      // {c(2t), c(2t+1)} x {row g, row g+8} the item loop starts from; an all-ones A gives sum x.
#pragma unroll
      for (int j = 0; j < (BITS == 4 ? KPW : 0); ++j)
#pragma unroll
        for (int h = 0; h < TE; ++h) {
          constexpr uint32_t L = 0xe408e408u, H = 0xd480d480u, ONE = 0x3c003c00u;  // half2 of -1032, -72, 1
          float cf[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int st = (TWO ? 2 * h : 0); st < (TWO ? 2 * h + 2 : STEPS); ++st) {
            const uint4 v = xr[j][st];
            mma_16816(cf, L, L, H, H, v.x, v.y);
            mma_16816(cf, L, L, H, H, v.z, v.w);
            if constexpr (HAS_ZERO) {
              mma_16816(sf, ONE, ONE, ONE, ONE, v.x, v.y);
              mma_16816(sf, ONE, ONE, ONE, ONE, v.z, v.w);
            }
          }
          if (g == 0) {
            float *e = reinterpret_cast<float *>(smem_raw + p.tab_off + (size_t(warp) * (KPW * TE) + j * TE + h) * 128 + t * 32);
            e[0] = cf[0]; e[1] = cf[1]; e[2] = cf[2]; e[3] = cf[3]; e[4] = sf[0]; e[5] = sf[1];
          }
        }
#pragma unroll
      for (int j = 0; j < (BITS == 4 ? KPW : 0); ++j)
#pragma unroll
        for (int st = 0; st < STEPS; ++st) {
          xr[j][st].y = hmul2_rn(xr[j][st].y, 0x2c002c00u);  // half2(1/16, 1/16); exact unless |x| < 2^-10
          xr[j][st].w = hmul2_rn(xr[j][st].w, 0x2c002c00u);
        }
      __syncwarp();
      MGV_TRACE_MARK(1);
      first_round = false;
    }
    for (; filled < D; ++filled) issue(ring + filled * SLOT, filled < n);

    uint32_t slot = ring;
    int done = 0;
    for (int tl = 0; tl < ntl; ++tl) {
      static_for<0, KPW>([&](auto j_c) {
        constexpr int J = decltype(j_c)::value;
        cp_async_wait_fixed<D - 1>();  // the oldest group, i.e. this item, has landed
        if constexpr (BITS == 4) xreg_compute4<HAS_ZERO, TWO>(slot + w_lane, slot + s_lane, tab_lane + J * (TE * 128), xr[J], acc);
        else xreg_compute8<HAS_ZERO, TWO>(slot + w_lane, slot + s_lane, xr[J], acc);
        issue(slot, done + D < n);  // refill the slot just consumed
        ++done;
        slot += SLOT;
        if (slot == ring_end) slot = ring;
      });
      flush_acc<BITS, VAR_MMA, 8>(part + size_t(tl) * slot_floats + warp * n_out, acc, M, g, t);
    }
    cp_async_wait_fixed<0>();
    MGV_TRACE_MARK(3);
    __syncthreads();
    MGV_TRACE_MARK(4);
    for (int e = threadIdx.x; e < ntl * n_out; e += THREADS) {
      const int tile = e / n_out, i = e - tile * n_out;
      const float *src = part + size_t(tile) * slot_floats + i;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < NW; ++w) v += src[w * n_out];
      store_out<TILE_ROWS>(p, ta + tile, i, v);
    }
    if (tb < t_end) __syncthreads();  // part is reused by the next round
    MGV_TRACE_MARK(6);
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

struct Plan {
  int variant, mb, bits, has_zero;
  int tile_rows, tiles, ipt, total_tiles;
  int grid, blocks_per_sm, slots, smem, depth, ring_off, slot_bytes, xstep, nw, magic, tab_off, deal_base, deal_rem, batch, xs_off, xs_pitch;
  int align_tiles, split_tiles, gshift, two_groups, group, ki;
  int lean;  // the steady-state kernel of the common decode case takes the call
  int xreg;  // ... in its form with x in registers: k ranges per warp and tile (2 or 4), else 0
  size_t ws_counter_bytes, ws_bytes;
};

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
    if (const char *force = getenv("MGV_ITEM")) {  // tuning aid
      if (atoi(force) == 128) pl.ki = 128;
      if (atoi(force) == 256 && variant == MGV_VARIANT_MMA && group >= 128 && a.K % 128 == 0) pl.ki = 256;
    }
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
  if (const char *force = getenv("MGV_DEAL")) {  // tuning aid: "items" or "tiles" overrides the estimate
    if (!strcmp(force, "items")) split = have_ws_hint && pl.split_tiles > 0;
    if (!strcmp(force, "tiles")) split = false;
  }
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
    if (const char *force = getenv("MGV_DEAL")) {
      if (!strcmp(force, "pairs")) use_pairs = true;
      if (!strcmp(force, "tiles")) use_pairs = false;
    }
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
  const int fit = (dev.smem_optin - 2048 - pl.ring_off) / (NWARP * item_bytes);  // 1 KB static + 1 KB read-past pad
  if (fit < 1) return fail(MGV_STATUS_UNSUPPORTED, "gemv: shared memory cannot hold one item per warp for this shape");
  pl.depth = int(std::max<long long>(1, std::min<long long>(std::min(fit, MAX_DEPTH), items_per_warp)));
  // + 1 KB: lanes without a batch column read (and ignore) up to 1 KB past their slot's x area
  pl.smem = pl.ring_off + pl.depth * NWARP * item_bytes + 1024;
  // ---- the steady-state kernel (gemv_lean_kernel) where its preconditions hold ----
  pl.lean = 0;
  const int lean_nw = 16;  // 24 and 32 warps were measured slower: their rings are shallower
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
    // x in registers instead of shared memory: K = 4096 or 8192, 4-bit weights.  Measured at least
    // as fast as the staged form for M = 1 and up to 1.7x faster for batches (C3 M=8: 64 -> 37 us).
    const int kpw = pl.ipt % lean_nw == 0 ? pl.ipt / lean_nw : 0;
    // (a block with a single tile and M = 1 is quicker with x staged: C4 O-proj 4.2 against 4.6 us)
    bool use_xreg = (kpw == 2 || kpw == 4) && (a.M > 1 || tiles_per_block >= 2);
    if (const char *force = getenv("MGV_XREG")) use_xreg = (kpw == 2 || kpw == 4) && atoi(force) != 0;  // tuning aid: 0 keeps x staged
    pl.xreg = 0;
    if (use_xreg) {
      const int te = two ? 2 : 1;
      const int tab_x = pl.bits == 4 ? lean_nw * kpw * te * 128 : 0;
      const int avail = dev.smem_optin - 2048 - tab_x;
      const int ring_unit = lean_nw * slot;
      long long sl = (avail - 3 * ring_unit) / part_tile;  // room for the partial sums beside a ring of depth 3
      sl = std::max<long long>(1, std::min<long long>(sl, tiles_per_block));
      // Ring depth: measured on B200, a shallow ring wins -- three items per warp in flight, two where a
      // warp has six items or fewer in all (C2 6.42 / 6.66 / 6.75 / 6.78 us at depth 2 / 3 / 4 / 5, C5 gate/up
      // 41.2 / 38.6 / 38.7 / 39.6): more requests in flight only queue behind one another.
      int depth = int(std::min<long long>(items_per_warp <= 6 ? 2 : 3, (avail - sl * part_tile) / ring_unit));
      if (const char *cap = getenv("MGV_DEPTH")) depth = std::max(1, std::min<int>(atoi(cap), int((avail - sl * part_tile) / ring_unit)));  // tuning aid
      if (depth >= 1) {
        pl.lean = 1;
        pl.xreg = kpw;
        pl.nw = lean_nw;
        pl.two_groups = two;
        pl.magic = pl.bits == 4 ? 1 : 0;
        pl.slots = int(sl);
        pl.tab_off = int((sl * part_tile + 127) / 128 * 128);
        pl.xs_off = -1;
        pl.ring_off = pl.tab_off + tab_x;
        pl.xstep = 0;
        pl.depth = depth;
        pl.slot_bytes = slot;
        pl.smem = pl.ring_off + depth * ring_unit;
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
      if (const char *cap = getenv("MGV_DEPTH")) pl.depth = std::max(1, std::min(lean_fit, atoi(cap)));  // tuning aid
      pl.slot_bytes = slot;
      pl.smem = ring_off + pl.depth * lean_nw * slot;
    }
  }
  return MGV_STATUS_OK;
}

// Long items first; if their slots do not fit shared memory for this shape, short ones.
mgv_status make_plan(const mgv_gemv_args &a, const DeviceInfo &dev, bool have_ws_hint, Plan &pl) {
  const char *lean_env = getenv("MGV_LEAN");  // tuning aid: MGV_LEAN=0 keeps the general kernel
  if (!(lean_env && atoi(lean_env) == 0) && !getenv("MGV_ITEM")) {
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

template <auto KERN>
mgv_status launch_configured(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  MGV_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {  // allow the device's full dynamic shared memory, once per kernel and device
    int optin = 0;
    cudaFuncAttributes fa;
    MGV_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    MGV_CUDA_TRY(cudaFuncGetAttributes(&fa, KERN));
    MGV_CUDA_TRY(cudaFuncSetAttribute(KERN, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - int(fa.sharedSizeBytes)));
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3(pl.nw * 32);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  int n_attrs = 0;
  if (pl.align_tiles == 2) {  // pairs of blocks: clusters of two
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = 2;
    attrs[n_attrs].val.clusterDim.y = 1;
    attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  if (p.flags & MGV_FLAG_PDL) {  // may start before the previous kernel of the stream has finished
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++n_attrs;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n_attrs;
  MGV_CUDA_TRY(cudaLaunchKernelEx(&cfg, KERN, p));
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}

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

template <int BITS, bool HZ, bool TWO, int KPW>
mgv_status launch_xreg_depth(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  switch (pl.depth) {
    case 1: return launch_configured<gemv_xreg_kernel<BITS, HZ, TWO, 1, KPW>>(p, pl, s);
    case 2: return launch_configured<gemv_xreg_kernel<BITS, HZ, TWO, 2, KPW>>(p, pl, s);
    case 3: return launch_configured<gemv_xreg_kernel<BITS, HZ, TWO, 3, KPW>>(p, pl, s);
    case 4: return launch_configured<gemv_xreg_kernel<BITS, HZ, TWO, 4, KPW>>(p, pl, s);
    case 5: return launch_configured<gemv_xreg_kernel<BITS, HZ, TWO, 5, KPW>>(p, pl, s);
    case 6: return launch_configured<gemv_xreg_kernel<BITS, HZ, TWO, 6, KPW>>(p, pl, s);
    default: return fail(MGV_STATUS_CUDA_ERROR, "internal: no x-in-registers kernel of ring depth %d", pl.depth);
  }
}

template <int BITS, bool HZ>
mgv_status launch_xreg(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.xreg == 2) return pl.two_groups ? launch_xreg_depth<BITS, HZ, true, 2>(p, pl, s) : launch_xreg_depth<BITS, HZ, false, 2>(p, pl, s);
  return pl.two_groups ? launch_xreg_depth<BITS, HZ, true, 4>(p, pl, s) : launch_xreg_depth<BITS, HZ, false, 4>(p, pl, s);
}

template <int BITS, bool HZ>
mgv_status launch_lean(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  if (pl.xreg) return launch_xreg<BITS, HZ>(p, pl, s);
  return pl.two_groups ? launch_lean_nw<BITS, HZ, true>(p, pl, s) : launch_lean_nw<BITS, HZ, false>(p, pl, s);
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
  if (pl.lean) return launch_lean<BITS, HZ>(p, pl, s);
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

static bool split_batch(const mgv_gemv_args *a, DeviceInfo *dev);

extern "C" mgv_status mgv_gemv_launch_info(const mgv_gemv_args *a, mgv_launch_info *info) {
  if (!info) return fail(MGV_STATUS_INVALID_ARGUMENT, "launch_info: null info");
  Plan pl{};
  DeviceInfo *dev = nullptr;
  mgv_status st = plan_for(a, pl, &dev);
  if (st != MGV_STATUS_OK) return st;
  if (split_batch(a, dev)) {  // two launches: the first one's geometry is reported
    mgv_gemv_args lo = *a;
    lo.M = 8;
    pl = Plan{};
    if ((st = plan_for(&lo, pl, &dev)) != MGV_STATUS_OK) return st;
  }
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

// Batches of 9..16 rows whose first eight rows would run on a steady-state kernel are served as
// two launches (rows 0..7, rows 8..M-1): twice the weight traffic, but both passes at the
// steady-state kernels' rate, and the second finds part of the weights in L2 -- measured faster
// than the one general-kernel launch with x travelling in the ring (C3 M=16).  Not with peers or
// waits (their counts are per launch), batched problems, or MGV_BATCH_SPLIT=0.
static bool split_batch(const mgv_gemv_args *a, DeviceInfo *dev) {
  if (!a || a->M <= 8 || a->M > 16 || a->n_peers || a->wait_flag || (a->batch_count > 1)) return false;
  if (a->variant == MGV_VARIANT_SIMT) return false;
  if (const char *e = getenv("MGV_BATCH_SPLIT")) {
    if (atoi(e) == 0) return false;
  }
  mgv_gemv_args h = *a;
  h.M = 8;
  Plan pl{};
  return make_plan(h, *dev, h.workspace != nullptr, pl) == MGV_STATUS_OK && pl.lean;
}

extern "C" mgv_status mgv_gemv(const mgv_gemv_args *a, mgv_stream_t s) {
  Plan pl{};
  DeviceInfo *dev = nullptr;
  mgv_status st = plan_for(a, pl, &dev);
  if (st != MGV_STATUS_OK) return st;
  if (split_batch(a, dev)) {
    const size_t esz = (a->flags & MGV_FLAG_OUT_F32_PARTIAL) ? 4 : 2;
    mgv_gemv_args lo = *a, hi = *a;
    lo.M = 8;
    hi.M = a->M - 8;
    hi.x = static_cast<const char *>(a->x) + size_t(8) * a->ldx * 2;
    hi.out = static_cast<char *>(a->out) + size_t(8) * a->ldd * esz;
    if ((st = mgv_gemv(&lo, s)) != MGV_STATUS_OK) return st;
    return mgv_gemv(&hi, s);
  }
  GemvParams p{};
  p.w = static_cast<const uint8_t *>(a->weights);
  p.x = static_cast<const __half *>(a->x);
  p.scale = static_cast<const __half *>(a->scale);
  p.zero = pl.has_zero ? static_cast<const __half *>(a->zero) : nullptr;
  p.bias = (a->flags & MGV_FLAG_OUT_F32_PARTIAL) ? nullptr : static_cast<const __half *>(a->bias);
  p.out = a->out;
  p.ws_counters = static_cast<int *>(a->workspace);
  p.ws_slots = a->workspace ? reinterpret_cast<float *>(static_cast<uint8_t *>(a->workspace) + pl.ws_counter_bytes) : nullptr;
  p.ldx = a->ldx; p.ldd = a->ldd;
  p.bs_w = a->batch_stride_weights; p.bs_x = a->batch_stride_x; p.bs_scale = a->batch_stride_scale;
  p.bs_bias = a->batch_stride_bias; p.bs_out = a->batch_stride_out;
  p.alpha = a->alpha; p.beta = a->beta;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.gshift = pl.gshift; p.two_groups = pl.two_groups; p.ki = pl.ki;
  p.tiles = pl.tiles; p.ipt = pl.ipt; p.total_tiles = pl.total_tiles;
  p.align_tiles = pl.align_tiles; p.slots = pl.slots; p.depth = pl.depth; p.ring_off = pl.ring_off; p.slot_bytes = pl.slot_bytes; p.xstep = pl.xstep; p.xs_off = pl.xs_off; p.xs_pitch = pl.xs_pitch;
  p.tab_off = pl.tab_off; p.deal_base = pl.deal_base; p.deal_rem = pl.deal_rem; p.batch = pl.batch; p.flags = a->flags;
  p.wait_flag = static_cast<const unsigned *>(a->wait_flag);
  p.wait_state = static_cast<unsigned long long *>(a->wait_state);
  p.wait_delta = a->wait_delta;
  p.n_peers = a->n_peers;
  for (int q = 0; q < a->n_peers; ++q) {
    p.peer_out[q] = a->peer_out[q];
    p.peer_flag[q] = static_cast<unsigned *>(a->peer_flag[q]);
  }
  // ring slots filled before the wait for the previous kernel: measured best on B200 -- 4-bit: 3 (C2 7.2 / 6.8 / 7.3 /
  // 7.5 us at 2 / 3 / 4 / 5); 8-bit: 2 (C1 5.16 against 5.30 us at 3)
  p.prefill = pl.bits == 8 ? 2 : 3;
  if (const char *force = getenv("MGV_PREFILL")) p.prefill = std::max(0, atoi(force));  // tuning aid
  if (pl.bits == 4) return pl.has_zero ? dispatch_family<4, true>(p, pl, s) : dispatch_family<4, false>(p, pl, s);
  return pl.has_zero ? dispatch_family<8, true>(p, pl, s) : dispatch_family<8, false>(p, pl, s);
}

#ifdef MGV_TRACE
extern "C" int mgv_debug_read_trace(unsigned long long *dst) {
  return int(cudaMemcpyFromSymbol(dst, g_trace, sizeof(g_trace)));
}
#endif

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
  mgv_gemv_args b = *a;
  b.workspace = nullptr;
  b.workspace_bytes = 0;
  size_t need = 0;
  mgv_status st = mgv_gemv_workspace_size(&b, &need);
  if (st != MGV_STATUS_OK) return st;
  if (need > kStaticScratchBytes)
    return fail(MGV_STATUS_WORKSPACE_TOO_SMALL,
                "gemv_static_scratch: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu; "
                "use mgv_gemv with caller-owned scratch",
                need, kStaticScratchBytes);
  void *scratch = nullptr;
  if ((st = static_scratch_address(&scratch)) != MGV_STATUS_OK) return st;
  if (need) {
    // The array keeps whatever the previous call left.  Only the per-tile arrival counters at its
    // start must read zero when a launch begins; the slots behind them are written before they are read.
    const size_t tiles = size_t((b.N + (b.weight_bits == 4 ? 32 : 16) - 1) / (b.weight_bits == 4 ? 32 : 16)) *
                         size_t(b.batch_count <= 0 ? 1 : b.batch_count);
    MGV_CUDA_TRY(cudaMemsetAsync(scratch, 0, (tiles * 4 + 255) / 256 * 256, s));
    b.workspace = scratch;
    b.workspace_bytes = kStaticScratchBytes;
  }
  return mgv_gemv(&b, s);
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
