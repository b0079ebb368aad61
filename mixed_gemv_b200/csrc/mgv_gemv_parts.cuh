// Pieces shared by the GEMV translation units: the kernel parameter block, the host-side plan,
// the launch helper and the device helpers (conversion, cp.async, epilogue, output exchange).
#pragma once

#include <mutex>
#include <type_traits>

#include <cuda.h>  // CUtensorMap (types only: the encoder is looked up at run time)

#include "mgv_common.cuh"

namespace mgv {

// An item is KI = 128 or 256 consecutive k of a row tile (a kernel template parameter): 256 halves
// the per-item bookkeeping for shapes with enough items, 128 keeps small calls balanced.
constexpr int RG = 8;                   // row groups per tile
constexpr int MAX_DEPTH = 8;            // deepest per-warp prefetch ring
constexpr int VAR_SIMT = 1, VAR_MMA = 2;
constexpr int kSlotFloats = 16 * 32;    // largest batch bucket x largest tile: one scratch slot size for all kernels
constexpr int kMaxBlocksPerSM = 4;      // scratch is sized for this many resident blocks per SM

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
  const unsigned *wait_flag;            // this GPU's arrival counters, one per source MGV_COUNTER_STRIDE bytes apart (or null)
  unsigned long long *wait_state;       // launches that used this wait so far
  unsigned wait_delta;                  // arrivals one earlier launch of the chain brings FROM EACH source
  unsigned wait_sources;                // bit s: the kernel waits for the counter of source s
  int *err_word;                        // device error word of this GPU: bounded waits that give up OR a code into it
  const uint8_t *prefetch;              // memory a later call will read (normally the next layer's weights), or null
  size_t prefetch_bytes;
  int hint_late;                        // 1: the prefetch hint is issued after x has arrived instead of before the wait
  int bar_off;                          // first ring fill by tiled bulk copies: byte offset of its mbarriers, or 0
  alignas(64) CUtensorMap w_map;        // ... and the tiled view of the weights it copies from (see encode_weight_map)
};

template <int BITS>
struct Geometry {
  static constexpr int RPG = 16 / BITS;  // rows per 16-byte unit
  static constexpr int TILE_ROWS = RG * RPG;
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
// wait_arrived: lane s of the first warp polls the counter of source s (bounded, about a second),
// then the block meets.  One counter PER SOURCE: with a single summed counter a peer that runs a
// call ahead could make up for another peer's arrival that is still in flight.
__device__ __forceinline__ void wait_arrived(const GemvParams &p, unsigned target) {
  if (threadIdx.x < 32) {
    const unsigned *flag = p.wait_flag + threadIdx.x * (MGV_COUNTER_STRIDE / 4);
    bool done = ((p.wait_sources >> threadIdx.x) & 1u) == 0;
    const uint64_t t0 = global_timer_ns();
    while (!done) {
      for (int i = 0; i < 64 && !done; ++i) {
        unsigned v;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        done = int(v - target) >= 0;
      }
      if (!done && global_timer_ns() - t0 > 1000000000ull) {
        atomicOr(p.err_word, 0x40);
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

// The epilogue's parameters in registers.  Read from the constant bank one after the other, each
// behind the branch that needs it, they cost a block about 0.15 us at its very end; fetched
// together before the block's last barrier they cost nothing.  plain(): fp16 output of one problem
// without peers or the gated form -- the case store() serves itself; everything else goes through
// store_out.
struct EpilogueRegs {
  int flags, N;
  bool simple;
  float alpha, beta;
  const __half *bias;
  __half *out;
  int64_t ldd;
  __device__ __forceinline__ explicit EpilogueRegs(const GemvParams &p)
      : flags(p.flags), N(p.N),
        simple(!(p.flags & (MGV_FLAG_GATED_SILU | MGV_FLAG_OUT_F32_PARTIAL)) && p.n_peers == 0 && p.total_tiles == p.tiles),
        alpha(p.alpha), beta(p.beta), bias(p.bias), out(static_cast<__half *>(p.out)), ldd(p.ldd) {
    asm volatile("" ::"r"(flags), "r"(N), "r"(int(simple)), "f"(alpha), "f"(beta), "l"(bias), "l"(out), "l"(ldd));
  }
  // the bias of output row n (0 without a bias): callers fetch it before the barrier
  __device__ __forceinline__ float bias_of(int n) const { return (simple && bias && n < N) ? __half2float(bias[n]) : 0.0f; }
  template <int TILE_ROWS>
  __device__ __forceinline__ void store(const GemvParams &p, int tile, int i, float v, float b) const {
    if (!simple) {
      store_out<TILE_ROWS>(p, tile, i, v);
      return;
    }
    const int m = i / TILE_ROWS, n = tile * TILE_ROWS + i % TILE_ROWS;
    if (n >= N) return;
    out[size_t(m) * ldd + n] = __float2half_rn(apply_act(alpha * v + beta * b, flags));
  }
};

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

// The caller's prefetch hint: every block asks the L2 cache for its 1/grid share of the range
// (normally the next layer's weights), cut into 16 pieces issued by the first lane of each of 16
// warps.  Issued once the block's own first copies are on their way, so HBM keeps streaming
// through this call's wait for its predecessor, its arithmetic and the start of its successor.
__device__ __forceinline__ void prefetch_hint(const GemvParams &p) {
  if (p.prefetch_bytes == 0) return;
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) != 0 || warp >= 16) return;
  const size_t pieces = size_t(gridDim.x) * 16;
  const size_t piece = ((p.prefetch_bytes + pieces - 1) / pieces + 127) / 128 * 128;
  const size_t lo = (size_t(blockIdx.x) * 16 + warp) * piece;
  if (lo >= p.prefetch_bytes) return;
  const size_t len = min(piece, p.prefetch_bytes - lo) & ~size_t(15);
  for (size_t off = 0; off < len; off += 16384) {
    const uint32_t n = uint32_t(min(size_t(16384), len - off));
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.prefetch + lo + off), "r"(n) : "memory");
  }
}

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

// ---- copies of one item, every offset an immediate --------------------------------------
// wd, sd: the lane's weight / scale position in slot 0 of its ring; DOFF: byte offset of the
// slot; wp: the lane's weight pointer at k range 0 of the tile; WOFF: byte offset of the k range.
template <int SB, bool HAS_ZERO, bool TWO, int DOFF, int WOFF>
__device__ __forceinline__ void tile_copy_item(uint32_t wd, const uint8_t *wp, uint32_t sd, const __half *sp, const __half *zp,
                                               uint32_t n_col_bytes) {
  asm volatile(
      "cp.async.cg.shared.global [%0+%2], [%1+%6], 16;\n\t"
      "cp.async.cg.shared.global [%0+%3], [%1+%7], 16;\n\t"
      "cp.async.cg.shared.global [%0+%4], [%1+%8], 16;\n\t"
      "cp.async.cg.shared.global [%0+%5], [%1+%9], 16;" ::"r"(wd),
      "l"(wp), "n"(DOFF), "n"(DOFF + 512), "n"(DOFF + 1024), "n"(DOFF + 1536), "n"(WOFF), "n"(WOFF + 64), "n"(WOFF + 128),
      "n"(WOFF + 192)
      : "memory");
  asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(sp), "n"(DOFF), "n"(SB) : "memory");
  if constexpr (TWO) {
    const __half *sp2 = reinterpret_cast<const __half *>(reinterpret_cast<const uint8_t *>(sp) + n_col_bytes);
    asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(sp2), "n"(DOFF + 32 * SB), "n"(SB) : "memory");
  }
  if constexpr (HAS_ZERO) {
    constexpr int ZO = (TWO ? 64 : 32) * SB;
    asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(zp), "n"(DOFF + ZO), "n"(SB) : "memory");
    if constexpr (TWO) {
      const __half *zp2 = reinterpret_cast<const __half *>(reinterpret_cast<const uint8_t *>(zp) + n_col_bytes);
      asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(zp2), "n"(DOFF + ZO + 32 * SB), "n"(SB) : "memory");
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// ---- mbarrier and tiled bulk copy (TMA), for the first ring fill of the x-in-registers kernel ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One item of the weights: box (64 bytes, 8 row groups, 4 steps) at (0, row group, step) of the map,
// into 2 KB of shared memory at dst (128-byte aligned) of this block alone; bytes are counted on bar.
__device__ __forceinline__ void bulk_item(uint32_t dst, const CUtensorMap *map, int row_group, int step, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(row_group), "r"(step), "r"(bar)
               : "memory");
}
// Waits for the phase of the given parity, for at most about a second; then records the failure
// in the device error word and carries on (wrong sums, no hang).
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int *err_word) {
  uint32_t ok = 0;
  for (int i = 0; i < 1024 && !ok; ++i)
    asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.b32 %0, 1, 0, q;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
  if (ok) return;
  const uint64_t t0 = global_timer_ns();
  while (!ok) {
    for (int i = 0; i < 256 && !ok; ++i)
      asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.b32 %0, 1, 0, q;\n\t}"
                   : "=r"(ok)
                   : "r"(bar), "r"(parity)
                   : "memory");
    if (!ok && global_timer_ns() - t0 > 1000000000ull) {
      atomicOr(err_word, 0x80);
      return;
    }
  }
}

// The scales (and zeros) of one item alone, closed by the commit of the group: the form of
// tile_copy_item for an item whose weights travel by a tiled bulk copy.
template <int SB, bool HAS_ZERO, bool TWO, int DOFF>
__device__ __forceinline__ void tile_copy_scales(uint32_t sd, const __half *sp, const __half *zp, uint32_t n_col_bytes) {
  asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(sp), "n"(DOFF), "n"(SB) : "memory");
  if constexpr (TWO) {
    const __half *sp2 = reinterpret_cast<const __half *>(reinterpret_cast<const uint8_t *>(sp) + n_col_bytes);
    asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(sp2), "n"(DOFF + 32 * SB), "n"(SB) : "memory");
  }
  if constexpr (HAS_ZERO) {
    constexpr int ZO = (TWO ? 64 : 32) * SB;
    asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(zp), "n"(DOFF + ZO), "n"(SB) : "memory");
    if constexpr (TWO) {
      const __half *zp2 = reinterpret_cast<const __half *>(reinterpret_cast<const uint8_t *>(zp) + n_col_bytes);
      asm volatile("cp.async.ca.shared.global [%0+%2], [%1], %3;" ::"r"(sd), "l"(zp2), "n"(DOFF + ZO + 32 * SB), "n"(SB) : "memory");
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// base + a 32-bit byte offset as ONE multiply-add on the FMA pipe (a 64-bit add would be two
// integer-pipe instructions, and the integer pipe is the one that is short)
__device__ __forceinline__ const __half *ptr_plus(const __half *base, uint32_t bytes) {
  uint64_t r;
  asm("mad.wide.u32 %0, %1, 1, %2;" : "=l"(r) : "r"(bytes), "l"(reinterpret_cast<uint64_t>(base)));
  return reinterpret_cast<const __half *>(r);
}

// D = A*B with a zero accumulator input (no register is cleared for it)
__device__ __forceinline__ void mma_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}


// ------------------------------------------------------------------------------------------
// host side, shared by the translation units
// ------------------------------------------------------------------------------------------

struct Plan {
  int variant, mb, bits, has_zero;
  int tile_rows, tiles, ipt, total_tiles;
  int grid, blocks_per_sm, slots, smem, depth, ring_off, slot_bytes, xstep, nw, magic, tab_off, deal_base, deal_rem, batch, xs_off, xs_pitch;
  int align_tiles, split_tiles, gshift, two_groups, group, ki;
  int lean;  // the steady-state kernel of the common decode case takes the call
  int xreg;  // ... in its form with x in registers: k ranges per warp and tile (1..4), else 0
  int tile_dt;  // x in registers: whole tiles each warp keeps in flight (ring depth = xreg * tile_dt)
  int batch_kernel;  // M = 9..16 in one pass (mgv_gemv_batch.cu); xreg holds its k ranges per warp
  int tensor_fill;   // x in registers: the first ring fill travels by tiled bulk copies (cp.async.bulk.tensor)
  int bar_off;
  size_t ws_counter_bytes, ws_bytes;
};

// Launches KERN with the plan's grid, block and dynamic shared memory.  The first launch of each
// kernel on each device lifts its dynamic shared-memory limit to the device's opt-in maximum.
template <auto KERN>
mgv_status launch_configured(const GemvParams &p, const Plan &pl, cudaStream_t s) {
  static bool configured[64];
  static std::mutex mu;
  int dev = 0;
  MGV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MGV_STATUS_UNSUPPORTED, "gemv: device index %d beyond 63", dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[dev]) {
      int optin = 0;
      cudaFuncAttributes fa;
      MGV_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
      MGV_CUDA_TRY(cudaFuncGetAttributes(&fa, KERN));
      MGV_CUDA_TRY(cudaFuncSetAttribute(KERN, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - int(fa.sharedSizeBytes)));
      configured[dev] = true;
    }
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

// The steady-state kernels (mgv_gemv_fast.cu): dispatch on weight width, zeros, group size, x
// source and ring depth as the plan says.
mgv_status launch_fast(const GemvParams &p, const Plan &pl, cudaStream_t s);
// The x-in-registers kernel (mgv_gemv_tile.cu): K = 16 * 128 * pl.xreg.
mgv_status launch_tile(const GemvParams &p, const Plan &pl, cudaStream_t s);
// The single-pass kernel for batches of 9..16 rows (mgv_gemv_batch.cu): K = 16 * 128 * pl.xreg.
mgv_status launch_batch(const GemvParams &p, const Plan &pl, cudaStream_t s);

}  // namespace mgv
