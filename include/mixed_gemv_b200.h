/*
 * mixed_gemv_b200 -- C ABI of the B200 (sm_100a) weight-only-quantised GEMV library.
 *
 *   D[m][n] = half( alpha * sum_k dequant(W[n][k]) * x[m][k]  +  beta * bias[n] )
 *   dequant(q) = half(half(q) * scale[g][n]) (+ zero[g][n]),  g = k / group_size
 *
 * Dimension names: M = batch rows of x (1..16), N = output features, K = reduction.
 * The reference calls N "M" and fixes its own "N" to 1 (mixed_gemv_test.cu:39,187).
 *
 * Every entry point takes plain pointers and sizes, returns an mgv_status and never
 * prints or exits (the reference prints and calls exit(-1): gemv/device/gemv_adaptor.h:199-203,
 * utils/preprocess.h:129-132).  All device pointers are caller-owned; except where a
 * function says otherwise nothing is allocated, and work is enqueued on the given stream
 * without synchronising.  Entry points are re-entrant; the only shared state is the
 * caller's workspace -- and, for mgv_gemv_static_scratch alone, the library's built-in scratch
 * array, which all calls on a device share (see there).  The library never reads the environment.
 *
 * Each declaration names the reference interface it stands in for (paths are relative to
 * the reference project's root).
 */
#ifndef MIXED_GEMV_B200_H_
#define MIXED_GEMV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ABI-compatible with cudaStream_t without pulling in the CUDA headers. */
typedef struct CUstream_st *mgv_stream_t;

typedef enum mgv_status {
  MGV_STATUS_OK = 0,
  MGV_STATUS_INVALID_ARGUMENT = 1,    /* null pointer, bad size, divisibility rule broken   */
  MGV_STATUS_UNSUPPORTED = 2,         /* well-formed but not implemented (e.g. W4_AFP8)     */
  MGV_STATUS_MISALIGNED = 3,          /* a pointer or leading dimension breaks an alignment */
  MGV_STATUS_WORKSPACE_TOO_SMALL = 4, /* the shape needs split-K scratch that was not given */
  MGV_STATUS_CUDA_ERROR = 5,          /* a CUDA runtime call failed; see mgv_last_error()   */
  MGV_STATUS_DEVICE_TIMEOUT = 6       /* a bounded device-side wait gave up                 */
} mgv_status;

/* gemv/weight_only_quant_op.h:12-18 -- same numeric values */
typedef enum mgv_quant_op {
  MGV_QUANT_UNDEFINED = 0,
  MGV_QUANT_PER_COLUMN_SCALE_ONLY = 1,
  MGV_QUANT_FINEGRAINED_SCALE_ONLY = 2,
  MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS = 3
} mgv_quant_op;

/* utils/type_base.h:7-11 -- same numeric values */
typedef enum mgv_quant_type { MGV_W8_A16 = 0, MGV_W4_A16 = 1, MGV_W4_AFP8 = 2 } mgv_quant_type;

/* utils/type_base.h:13-16 -- same numeric values */
typedef enum mgv_layout { MGV_LAYOUT_ROW_MAJOR = 0, MGV_LAYOUT_COLUMN_MAJOR = 1 } mgv_layout;

/* kernel family: the choice the reference makes with template parameters */
typedef enum mgv_variant {
  MGV_VARIANT_AUTO = 0, /* pick per shape                                                  */
  MGV_VARIANT_SIMT = 1, /* CUDA-core multiply-accumulate (M <= 4)                          */
  MGV_VARIANT_MMA = 2   /* tensor-core multiply-accumulate of the dequantised tile (M <= 16)*/
} mgv_variant;

enum {
  /* out is float [M][ldd] = alpha * accumulator; bias is not added, nothing is rounded to
   * fp16.  Used by the K-split sharding, where partial sums are reduced across GPUs. */
  MGV_FLAG_OUT_F32_PARTIAL = 1,
  /* epilogue activation applied to alpha*acc + beta*bias before the fp16 store: the
   * Activation slot of host::reference::MixedGemv (host/mixed_gemv.h:17-18,103). */
  MGV_FLAG_ACT_RELU = 2,
  MGV_FLAG_ACT_SILU = 4,
  /* Programmatic dependent launch: the kernel may be started while the previous kernel of the
   * stream is still draining, and prefetches weights and scales meanwhile; it reads x and writes
   * out (and the scratch) only after that kernel has completed, so stream order is kept for
   * everything a previous kernel can produce.  Weights, scales, zeros and bias must NOT be
   * written by the immediately preceding kernel.  No counterpart in the reference. */
  MGV_FLAG_PDL = 8,
  /* Fused gate/up layer of a gated MLP: weight rows 2i and 2i+1 are the gate and the up
   * projection of output feature i (the caller interleaves the two matrices row by row before
   * preprocessing; scales, zeros and bias interleave the same way).  The epilogue then stores
   * out[m][i] = half(silu(g) * u) with g, u = alpha*acc + beta*bias of the two rows: N/2 features
   * per batch row, ldd >= N/2.  Not with MGV_FLAG_OUT_F32_PARTIAL or the activation flags.
   * The step after the path in a decoder layer (the Activation slot of host/mixed_gemv.h:17-18
   * applied to a fused gate/up matrix); no counterpart in the reference's device code. */
  MGV_FLAG_GATED_SILU = 16
};

const char *mgv_status_string(int status);
/* Message of the calling thread's most recent non-OK status ("" if none). */
const char *mgv_last_error(void);
/* Library version, major*10000 + minor*100 + patch. */
int mgv_version(void);

/* ---- weight / zero-point preparation (runs on the GPU, results bit-exact with the host code) ---- */

/* SubBytePacker<int4b_t,int8_t>::pack, utils/preprocess.h:55-84.
 * n_unpacked int8 values in [-8,7] -> n_unpacked/2 bytes, even index in the low nibble. */
mgv_status mgv_pack_int4(void *dst_dev, const void *src_dev, size_t n_unpacked, mgv_stream_t s);

/* SubBytePacker<int4b_t,int8_t>::unpack, utils/preprocess.h:41-53 (sign-extends). */
mgv_status mgv_unpack_int4(void *dst_dev, const void *src_dev, size_t n_packed, mgv_stream_t s);

/* MixedGemvWeightPreprocessor::run, utils/preprocess.h:480-522: optional [K,N]->[N,K]
 * transpose (:123-290), row interleave (:292-362), +8/+128 bias and in-word element
 * permutation (:365-455), fused into one pass.  shape = {K,N} (rank 2) or {E,K,N} (rank 3).
 * dst and src hold shape-product * bits / 8 bytes and must not overlap.  W8_A16 follows the
 * reference's interleave template with a 64-bit access unit (its public dispatcher refuses
 * it, :353-361); W4_AFP8 returns MGV_STATUS_UNSUPPORTED as no kernel consumes it.
 * Preconditions (INVALID_ARGUMENT otherwise): N % (16/bits) == 0, K % 8 == 0, and for
 * MGV_LAYOUT_ROW_MAJOR both N*bits/8 and K*bits/8 multiples of 32 (:151-162). */
mgv_status mgv_preprocess_weights(void *dst_dev, const void *src_dev, const size_t *shape,
                                  int rank, int layout, int quant_type, mgv_stream_t s);

/* ZeroPointPreprocessor<half,int8_t>::neg_zero_point_multiplies_scale,
 * utils/preprocess.h:94-101: dst[i] = half(-zeros[i]) * scales[i]. */
mgv_status mgv_preprocess_zeros(void *dst_f16_dev, const void *scales_f16_dev,
                                const void *zeros_i8_dev, size_t n, mgv_stream_t s);

/* ---- the GEMV ---- */

/* Stands in for GemvAdaptor::Arguments, gemv/device/gemv_adaptor.h:114-178, as filled by
 * device_gemv(), mixed_gemv_test.cu:124-165. */
typedef struct mgv_gemv_args {
  int32_t struct_size; /* sizeof(mgv_gemv_args); guards against header/library skew          */
  int32_t M;           /* batch rows of x and out, 1..16                                      */
  int32_t N;           /* output features; multiple of 16/weight_bits                         */
  int32_t K;           /* reduction length; multiple of 64                                    */
  int32_t weight_bits; /* 4 or 8                                                              */
  int32_t quant_op;    /* mgv_quant_op                                                        */
  int32_t group_size;  /* power of two >= 64 dividing K; ignored (taken as K) per-column      */
  int32_t variant;     /* mgv_variant                                                         */
  int32_t flags;       /* MGV_FLAG_*                                                          */
  int32_t batch_count; /* independent problems, >= 1 (0 is read as 1); gemv_adaptor.h:130     */
  const void *weights; /* preprocessed weights, 16-byte aligned (ref_A; lda is implied)       */
  const void *x;       /* fp16 [M][ldx], 16-byte aligned (ref_B; the reference has ldb = 0)    */
  const void *scale;   /* fp16 [G][N], G = K/group_size (ref_scale, stride N)                 */
  const void *zero;    /* fp16 [G][N] additive zeros = -zero_point*scale, or NULL (ref_zero_point) */
  const void *bias;    /* fp16 [N] or NULL (ref_C, the epilogue source)                       */
  void *out;           /* fp16 [M][ldd] (ref_D), or float with MGV_FLAG_OUT_F32_PARTIAL       */
  int64_t ldx;         /* elements between batch rows of x; multiple of 8                     */
  int64_t ldd;         /* elements between batch rows of out                                  */
  float alpha;         /* epilogue: out = alpha*acc + beta*bias (LinearCombination)           */
  float beta;
  /* element strides between problems of a batch: gemv_adaptor.h:131-135 */
  int64_t batch_stride_weights; /* in BYTES of the preprocessed buffer                        */
  int64_t batch_stride_x;
  int64_t batch_stride_scale;   /* applies to scale and zero                                  */
  int64_t batch_stride_bias;
  int64_t batch_stride_out;
  void *workspace;        /* split-K scratch from mgv_gemv_workspace_size, or NULL            */
  size_t workspace_bytes;
  /* Output exchange of an N-split (sharded) layer, fused into the epilogue -- no counterpart in
   * the reference, which is single-GPU.  With n_peers > 0 every output element is stored to
   * `out` AND, at the same element offset, to each peer_out[i] (device pointers into other GPUs'
   * memory, mapped with mgv_window_open, laid out like `out`); when a thread block has stored
   * all its outputs it adds 1 to the 4-byte counter each peer_flag[i] points to (system scope,
   * after a system-wide fence), so a consumer that has seen `grid` arrivals of a launch
   * (mgv_gemv_launch_info) holds all of its output.  With MGV_FLAG_OUT_F32_PARTIAL the stores are
   * the fp32 partials (K-split layers; mgv_reduce_partials finishes them). */
  int32_t n_peers;        /* 0..MGV_MAX_PEERS                                                  */
  int32_t hints;          /* MGV_HINT_* (0: the library chooses)                               */
  void *peer_out[8];
  void *peer_flag[8];     /* entries may be NULL (no signal to that peer)                      */
  /* The consumer side of that exchange, inside the kernel.  A GPU keeps ONE 4-byte arrival
   * counter PER SOURCE, MGV_COUNTER_STRIDE bytes apart, in a window of its own: source s counts
   * in on counter s (its peer_flag for this GPU points there).  With wait_flag set to the base of
   * these counters, the kernel does not read x before every counter s with bit s of wait_sources
   * set has reached L * wait_delta -- L being the number of earlier launches that used the same
   * wait_state (an 8-byte counter in device memory, zero before the first launch; the kernel
   * counts itself in), wait_delta the arrivals ONE launch of ONE source brings (its grid).  So in
   * a chain of sharded layers launch L waits for the peers' slices of launches 0..L-1, and the
   * first launch waits for nothing.  All launches sharing a wait_state must have the same grid on
   * every GPU (equal shards) and run in stream order.  The wait is bounded like mgv_wait_arrivals.
   * (Per-source counters: with one summed counter a peer that runs a call ahead could stand in
   * for another peer's arrival that is still in flight.) */
  const void *wait_flag;
  void *wait_state;
  uint32_t wait_delta;
  uint32_t wait_sources;
  /* Prefetch hint -- no counterpart in the reference.  A range of device memory that a LATER call
   * on this GPU will read, normally the preprocessed weights of the next layer: once this call's
   * own first copies are on their way, its thread blocks ask the L2 cache to fetch the range
   * (cp.async.bulk.prefetch.L2), so HBM keeps streaming while this call waits for its
   * predecessor, computes and hands over, and the next call finds its first weights in L2.
   * Nothing is computed from the range and results never depend on it.  16-byte aligned; sensible
   * up to a quarter of the L2 (about 30 MB on B200) -- more evicts what this call still needs.
   * NULL / 0: no prefetch. */
  const void *prefetch;
  size_t prefetch_bytes;
} mgv_gemv_args;

#define MGV_MAX_PEERS 8
#define MGV_COUNTER_STRIDE 32 /* bytes between the per-source arrival counters of a GPU */

/* Plan hints (mgv_gemv_args.hints).  Every combination computes the same result through another
 * code path; they exist so that tests and tuning runs can reach each path on any shape.  A hint
 * whose preconditions do not hold for the shape is ignored. */
enum {
  MGV_HINT_DEAL_TILES = 1,     /* every thread block owns whole row tiles                        */
  MGV_HINT_DEAL_ITEMS = 2,     /* equal k ranges cut anywhere, combined through the scratch      */
  MGV_HINT_DEAL_PAIRS = 3,     /* clusters of two blocks halve a tile range (no scratch)         */
  MGV_HINT_ITEM_128 = 4,       /* k length of a work item of the general kernel                  */
  MGV_HINT_ITEM_256 = 8,
  MGV_HINT_KERNEL_GENERAL = 16, /* the general kernel even where a steady-state kernel applies   */
  MGV_HINT_KERNEL_STAGED = 32,  /* the steady-state kernel with x staged in shared memory        */
  MGV_HINT_KERNEL_XREG = 48,    /* the steady-state kernel with x in registers                   */
  MGV_HINT_ONE_LAUNCH = 64      /* M = 9..16: one launch, never rows 0..7 and 8..M-1 separately  */
};

/* Fills *args with defaults (struct_size, alpha = beta = 1, batch_count = 1, AUTO). */
void mgv_gemv_args_init(mgv_gemv_args *args);

/* Scratch the kernel may need to combine row tiles whose K range is split over thread blocks.
 * No counterpart in the reference, which never splits K across blocks
 * (gemv/threadblock/accumulator_combine.h:224-330 reduces inside one block only).
 * The size depends on M, N, K, weight_bits and the device only.  The scratch must be zeroed
 * once (mgv_workspace_init) before its first use; the kernel leaves it zeroed.  Two calls that
 * may overlap on the GPU must not share it.  The scratch is optional: without it every thread
 * block owns whole row tiles; with it the library cuts tiles between blocks when it estimates that
 * the better balance outweighs the combine step (MGV_HINT_DEAL_* overrides the estimate). */
mgv_status mgv_gemv_workspace_size(const mgv_gemv_args *args, size_t *bytes);
mgv_status mgv_workspace_init(void *workspace_dev, size_t bytes, mgv_stream_t s);

/* GemvAdaptor::initialize + run, gemv/device/gemv_adaptor.h:198-255.  Validates the
 * arguments, picks the kernel and enqueues ONE launch on `s` -- two for batches of 9..16 rows
 * where serving rows 0..7 and 8..M-1 separately on the steady-state kernels is faster (never
 * with peers, waits or batch_count > 1; MGV_HINT_ONE_LAUNCH forbids it). */
mgv_status mgv_gemv(const mgv_gemv_args *args, mgv_stream_t s);

/* The same in two steps, as GemvAdaptor::initialize (:198-223, builds Params once) and
 * GemvAdaptor::run (:226-255, launches only): mgv_gemv_plan_create validates the arguments, picks
 * the kernel and stores everything a launch needs (host memory only; pointers are captured, so the
 * buffers must stay where they are); mgv_gemv_plan_run enqueues the launch(es) with no further
 * host work than the launch itself.  A plan belongs to the device that was current when it was
 * made and may be run any number of times, also while a stream is being captured. */
typedef struct mgv_gemv_plan mgv_gemv_plan;
mgv_status mgv_gemv_plan_create(const mgv_gemv_args *args, mgv_gemv_plan **plan);
mgv_status mgv_gemv_plan_run(const mgv_gemv_plan *plan, mgv_stream_t s);
void mgv_gemv_plan_destroy(mgv_gemv_plan *plan);

/* mgv_gemv for callers that cannot allocate device memory -- no counterpart in the reference.
 * Who needs it: code that runs while a stream is being captured (cudaMalloc is forbidden there), an
 * inference-runtime plug-in whose enqueue hook gets a fixed memory budget, a real-time loop that
 * must stay off the allocator, a language binding with no device allocator at hand.  Same
 * arguments and results as mgv_gemv, except that args->workspace is ignored: the split-K scratch
 * is a 4 MiB array inside the library image (each GPU that loads the library holds it until the
 * process exits).  The call allocates nothing: no cudaMalloc, no cudaFree, no allocating library
 * routine.  Shapes whose scratch would exceed 4 MiB (about 400 000 row tiles) are refused with
 * MGV_STATUS_WORKSPACE_TOO_SMALL; use mgv_gemv with your own scratch for those.
 * The first call on each device looks the array's device address up (cudaGetSymbolAddress); make
 * that first call before any stream capture begins.  The address is cached per device ordinal for
 * the life of the process: after cudaDeviceReset the cached value is stale, do not call again.  All calls on a device share the one array:
 * the part that must start at zero is cleared on the stream at each call, but two calls that can
 * overlap on the GPU (different streams without ordering) race on it -- serialise them. */
mgv_status mgv_gemv_static_scratch(const mgv_gemv_args *args, mgv_stream_t s);

/* ---- memory windows and arrival counters for the fused output exchange ---- */

/* Allocates `bytes` of zeroed device memory on the current GPU that other processes of the node
 * can map, and writes its 64-byte inter-process handle to ipc_handle_64 (send it to the peers
 * by any host channel). */
mgv_status mgv_window_create(void **dev_ptr, size_t bytes, void *ipc_handle_64);
/* Maps a peer's window into this process (the current GPU must be able to reach the peer's GPU:
 * NVLink or PCIe peer access).  *peer_ptr is usable as peer_out / peer_flag in mgv_gemv_args. */
mgv_status mgv_window_open(const void *ipc_handle_64, void **peer_ptr);
mgv_status mgv_window_close(void *peer_ptr);
mgv_status mgv_window_destroy(void *dev_ptr);
/* Enqueues on `s` a one-warp kernel that returns when every arrival counter s of this GPU with
 * bit s of `sources` set (counters_dev + s * MGV_COUNTER_STRIDE, in a window of the current GPU)
 * has grown by `delta` beyond the 4-byte count at seen_dev (compared modulo 2^32: counters only
 * grow), then adds delta to *seen_dev -- so the same call can be replayed from a CUDA graph, one
 * replay per round of arrivals.  delta = arrivals one round brings from EACH source.
 * The wait is bounded (about one second); when it gives up it raises the device error word
 * (mgv_device_error_state reports MGV_STATUS_DEVICE_TIMEOUT), still adds delta, and returns, so
 * the stream never hangs on a peer that died.  The producers must run on OTHER GPUs (or earlier
 * on this one). */
mgv_status mgv_wait_arrivals(const void *counters_dev, void *seen_dev, uint32_t sources, uint32_t delta, mgv_stream_t s);

/* K-split (row-split) layers: every GPU holds `parts` fp32 partial outputs [M][ld_in], part r
 * starting part_stride_elems * r floats after the first (with the fused exchange: the slots of a
 * window that each GPU's kernel, run with MGV_FLAG_OUT_F32_PARTIAL and peers, filled).  Adds them
 * in order r = 0..parts-1, then out = half(act(sum + beta*bias)).  The final step of the
 * reference's epilogue (epilogue/threadblock/epilogue.h:78-97), applied once after the reduction. */
mgv_status mgv_reduce_partials(const void *partials_f32_dev, size_t part_stride_elems, int parts, int M, int N,
                               long long ld_in, const void *bias_f16_dev, float beta, int flags, void *out_f16_dev,
                               long long ld_out, mgv_stream_t s);

/* mgv_wait_arrivals and mgv_reduce_partials in ONE launch, for chains of K-split layers (the reference
 * has no counterpart: it is single-GPU).  Every thread block waits -- bounded, as above -- until each
 * counter s with bit s of `sources` set has reached (launches that used state_dev so far + 1) * delta,
 * then adds its share of the partials.  state_dev: 8 zeroed bytes in device memory that only calls of
 * one shape (M, N) share (it counts launches in units of their grid).  With MGV_FLAG_PDL in `flags`
 * the launch may start while the kernel before it on the stream drains and lets the kernel after it
 * start early; it waits for its predecessor before it polls or reads.  Other flags: the activations. */
mgv_status mgv_wait_reduce_partials(const void *partials_f32_dev, size_t part_stride_elems, int parts, int M, int N,
                                    long long ld_in, const void *bias_f16_dev, float beta, int flags, void *out_f16_dev,
                                    long long ld_out, const void *counters_dev, void *state_dev, uint32_t sources,
                                    uint32_t delta, mgv_stream_t s);

/* Reads (and clears) the device-side error word that bounded waits inside the kernels set
 * when they give up.  Synchronises the device.  *state receives 0 when no wait timed out. */
mgv_status mgv_device_error_state(int *state);

/* What mgv_gemv would launch for these arguments (no launch is made). */
typedef struct mgv_launch_info {
  int32_t variant;        /* resolved mgv_variant                     */
  int32_t grid;           /* thread blocks                            */
  int32_t block;          /* threads per block                        */
  int32_t stages;         /* shared-memory ring depth                 */
  int32_t smem_bytes;     /* dynamic shared memory per block          */
  int32_t tile_rows;      /* output rows per tile                     */
  int32_t k_slice;        /* K elements per stage                     */
  int32_t split_tiles;    /* row tiles combined across blocks         */
} mgv_launch_info;
mgv_status mgv_gemv_launch_info(const mgv_gemv_args *args, mgv_launch_info *info);

/* ---- a resident layer: the flow of main(), mixed_gemv_test.cu:245-283, behind one handle ----
 * These are the only entry points that allocate device memory. */

typedef struct mgv_linear mgv_linear;

/* Uploads un-preprocessed host weights ({K,N}, `layout`), preprocesses them on the GPU and
 * keeps weights, scales, additive zeros and bias resident on the current device.
 * zeros_f16_host and bias_f16_host may be NULL.  max_M bounds later forward calls. */
mgv_status mgv_linear_create(mgv_linear **out, int N, int K, int weight_bits, int quant_op,
                             int group_size, int layout, const void *weights_host,
                             const void *scale_f16_host, const void *zeros_f16_host,
                             const void *bias_f16_host, int max_M);

/* x_host fp16 [M][K] -> out_host fp16 [M][N]: copies x to the device, runs mgv_gemv, brings
 * the result back and waits for it.  Host buffers may be pageable or pinned.  With pinned
 * (page-locked, mapped) buffers the call replays a two-node CUDA graph -- a one-block kernel
 * that reads x over PCIe, and a GEMV launched as its programmatic dependent (it prefetches
 * weights meanwhile) whose epilogue writes the result straight into out_host -- rebuilt when
 * the buffers, M or the variant change; pageable buffers take two copies around the kernel. */
mgv_status mgv_linear_forward_host(mgv_linear *layer, const void *x_host, void *out_host, int M,
                                   int variant);

/* Device-pointer forward on a caller stream (no copies, no synchronisation). */
mgv_status mgv_linear_forward(mgv_linear *layer, const void *x_dev, void *out_dev, int M,
                              int variant, mgv_stream_t s);

const void *mgv_linear_weights(const mgv_linear *layer); /* preprocessed, device */
void mgv_linear_destroy(mgv_linear *layer);

#ifdef __cplusplus
}
#endif
#endif /* MIXED_GEMV_B200_H_ */
