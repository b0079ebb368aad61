// Memory windows and arrival counters for the output exchange of an N-split (sharded) layer.
//
// The reference is single-GPU.  When one layer is cut over the GPUs of a node along its output
// features, every GPU needs every other GPU's slice of the output before the next layer.  Here
// the GEMV's epilogue stores each output element straight into all GPUs' gather buffers (peer
// stores over NVLink) and counts its thread blocks in on a per-GPU arrival counter, so the
// exchange overlaps the kernel's tail and needs no collective call; what is left for the
// consumer is a bounded wait on its own counter.  This file holds the host plumbing: windows
// that other processes can map (CUDA IPC) and the wait.
#include <algorithm>
#include <cstring>

#include "mgv_common.cuh"

namespace mgv {

// Lane s of one warp polls the counter of source s with system-scope loads until it has grown by
// `delta` beyond *seen; then *seen moves on.  The wait is bounded by the global timer: a peer that
// never arrives costs about a second, raises the error word and lets the stream continue.
__global__ void wait_arrivals_kernel(const unsigned *counters, unsigned *seen, unsigned sources, unsigned delta, int *error_word) {
  const unsigned target = *seen + delta;
  __syncwarp();
  if (threadIdx.x == 0) *seen = target;
  if ((sources >> threadIdx.x) & 1u) {
    const unsigned *flag = counters + threadIdx.x * (MGV_COUNTER_STRIDE / 4);
    const uint64_t t0 = global_timer_ns();
    for (bool done = false; !done;) {
      for (int i = 0; i < 64 && !done; ++i) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        done = int(v - target) >= 0;
      }
      if (!done && global_timer_ns() - t0 > 1000000000ull) {
        atomicOr(error_word, 0x20);
        done = true;
      }
    }
  }
}

// K-split layers: out = half(act(sum over the `parts` fp32 partial outputs, in order) + beta*bias)
__global__ void reduce_partials_kernel(const float *partials, size_t part_stride, int parts, int M, int N, long long ld_in,
                                       const __half *bias, float beta, int flags, __half *out, long long ld_out) {
  const size_t total = size_t(M) * N;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int m = int(i / N), n = int(i - size_t(m) * N);
    float v = 0.0f;
    for (int r = 0; r < parts; ++r) v += __ldcg(partials + r * part_stride + size_t(m) * ld_in + n);
    if (bias) v += beta * __half2float(bias[n]);
    if (flags & MGV_FLAG_ACT_RELU) v = fmaxf(v, 0.0f);
    if (flags & MGV_FLAG_ACT_SILU) v = v / (1.0f + __expf(-v));
    out[size_t(m) * ld_out + n] = __float2half_rn(v);
  }
}

// The two in one launch, for a chain of K-split layers: every block counts the launch in (the
// launches that used `state` so far, times the blocks of one launch, give the round), lets the next
// kernel of the stream begin its set-up, waits for its own GPU's kernel before it (whose partial it
// reads) and then -- bounded -- for this round's arrivals from every source; then it adds its share.
__global__ void wait_reduce_partials_kernel(const float *partials, size_t part_stride, int parts, int M, int N, long long ld_in,
                                            const __half *bias, float beta, int flags, __half *out, long long ld_out,
                                            const unsigned *counters, unsigned long long *state, unsigned sources, unsigned delta,
                                            int *error_word) {
  __shared__ unsigned sh_target;
  if (threadIdx.x == 0) {
    const unsigned long long my = atomicAdd(state, 1ull);
    sh_target = unsigned((my / gridDim.x + 1ull) * delta);
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x < 32) {
    const unsigned target = sh_target;
    const unsigned *flag = counters + threadIdx.x * (MGV_COUNTER_STRIDE / 4);
    bool done = ((sources >> threadIdx.x) & 1u) == 0;
    const uint64_t t0 = global_timer_ns();
    while (!done) {
      for (int i = 0; i < 64 && !done; ++i) {
        unsigned v;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        done = int(v - target) >= 0;
      }
      if (!done && global_timer_ns() - t0 > 1000000000ull) {
        atomicOr(error_word, 0x20);
        done = true;
      }
    }
    asm volatile("fence.acquire.sys;" ::: "memory");  // what the counted blocks stored is visible from here on
  }
  __syncthreads();
  const size_t total = size_t(M) * N;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int m = int(i / N), n = int(i - size_t(m) * N);
    float v = 0.0f;
    for (int r = 0; r < parts; ++r) v += __ldcg(partials + r * part_stride + size_t(m) * ld_in + n);
    if (bias) v += beta * __half2float(bias[n]);
    if (flags & MGV_FLAG_ACT_RELU) v = fmaxf(v, 0.0f);
    if (flags & MGV_FLAG_ACT_SILU) v = v / (1.0f + __expf(-v));
    out[size_t(m) * ld_out + n] = __float2half_rn(v);
  }
}

}  // namespace mgv

using namespace mgv;

extern "C" mgv_status mgv_window_create(void **dev_ptr, size_t bytes, void *ipc_handle_64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the header promises a 64-byte handle");
  if (!dev_ptr || !ipc_handle_64 || bytes == 0) return fail(MGV_STATUS_INVALID_ARGUMENT, "window_create: null argument or zero size");
  *dev_ptr = nullptr;
  void *p = nullptr;
  MGV_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "window_create");
  }
  std::memcpy(ipc_handle_64, &h, sizeof(h));
  *dev_ptr = p;
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_window_open(const void *ipc_handle_64, void **peer_ptr) {
  if (!ipc_handle_64 || !peer_ptr) return fail(MGV_STATUS_INVALID_ARGUMENT, "window_open: null argument");
  *peer_ptr = nullptr;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, ipc_handle_64, sizeof(h));
  void *p = nullptr;
  MGV_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *peer_ptr = p;
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_window_close(void *peer_ptr) {
  if (!peer_ptr) return MGV_STATUS_OK;
  MGV_CUDA_TRY(cudaIpcCloseMemHandle(peer_ptr));
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_window_destroy(void *dev_ptr) {
  if (!dev_ptr) return MGV_STATUS_OK;
  MGV_CUDA_TRY(cudaFree(dev_ptr));
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_wait_arrivals(const void *counters_dev, void *seen_dev, uint32_t sources, uint32_t delta, mgv_stream_t s) {
  const void *flag_dev = counters_dev;
  if (!flag_dev || !seen_dev) return fail(MGV_STATUS_INVALID_ARGUMENT, "wait_arrivals: null counter");
  if (reinterpret_cast<uintptr_t>(flag_dev) % 4 || reinterpret_cast<uintptr_t>(seen_dev) % 4)
    return fail(MGV_STATUS_MISALIGNED, "wait_arrivals: the counters must be 4-byte aligned");
  int *err = device_error_word();
  if (!err) return fail(MGV_STATUS_CUDA_ERROR, "wait_arrivals: no device error word");
  wait_arrivals_kernel<<<1, 32, 0, static_cast<cudaStream_t>(s)>>>(static_cast<const unsigned *>(flag_dev),
                                                                   static_cast<unsigned *>(seen_dev), sources, delta, err);
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_reduce_partials(const void *partials_f32_dev, size_t part_stride_elems, int parts, int M, int N,
                                          long long ld_in, const void *bias_f16_dev, float beta, int flags, void *out_f16_dev,
                                          long long ld_out, mgv_stream_t s) {
  if (!partials_f32_dev || !out_f16_dev) return fail(MGV_STATUS_INVALID_ARGUMENT, "reduce_partials: null argument");
  if (parts < 1 || M < 1 || N < 1 || ld_in < N || ld_out < N) return fail(MGV_STATUS_INVALID_ARGUMENT, "reduce_partials: bad shape");
  if (flags & ~(MGV_FLAG_ACT_RELU | MGV_FLAG_ACT_SILU)) return fail(MGV_STATUS_INVALID_ARGUMENT, "reduce_partials: only activation flags apply");
  const size_t total = size_t(M) * N;
  const int blocks = int(std::min<size_t>((total + 255) / 256, 1024));
  reduce_partials_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(s)>>>(
      static_cast<const float *>(partials_f32_dev), part_stride_elems, parts, M, N, ld_in, static_cast<const __half *>(bias_f16_dev),
      beta, flags, static_cast<__half *>(out_f16_dev), ld_out);
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_wait_reduce_partials(const void *partials_f32_dev, size_t part_stride_elems, int parts, int M, int N,
                                               long long ld_in, const void *bias_f16_dev, float beta, int flags, void *out_f16_dev,
                                               long long ld_out, const void *counters_dev, void *state_dev, uint32_t sources,
                                               uint32_t delta, mgv_stream_t s) {
  if (!partials_f32_dev || !out_f16_dev || !counters_dev || !state_dev) return fail(MGV_STATUS_INVALID_ARGUMENT, "wait_reduce_partials: null argument");
  if (parts < 1 || M < 1 || N < 1 || ld_in < N || ld_out < N) return fail(MGV_STATUS_INVALID_ARGUMENT, "wait_reduce_partials: bad shape");
  if (flags & ~(MGV_FLAG_ACT_RELU | MGV_FLAG_ACT_SILU | MGV_FLAG_PDL))
    return fail(MGV_STATUS_INVALID_ARGUMENT, "wait_reduce_partials: only the activation flags and MGV_FLAG_PDL apply");
  if (reinterpret_cast<uintptr_t>(counters_dev) % 4 || reinterpret_cast<uintptr_t>(state_dev) % 8)
    return fail(MGV_STATUS_MISALIGNED, "wait_reduce_partials: counters 4-byte, state 8-byte aligned");
  int *err = device_error_word();
  if (!err) return fail(MGV_STATUS_CUDA_ERROR, "wait_reduce_partials: no device error word");
  const size_t total = size_t(M) * N;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(std::min<size_t>((total + 255) / 256, 148)));  // a function of M and N only: `state` counts in units of it
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(s);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & MGV_FLAG_PDL) ? 1 : 0;
  MGV_CUDA_TRY(cudaLaunchKernelEx(&cfg, wait_reduce_partials_kernel, static_cast<const float *>(partials_f32_dev), part_stride_elems, parts,
                                  M, N, ld_in, static_cast<const __half *>(bias_f16_dev), beta, flags & ~MGV_FLAG_PDL,
                                  static_cast<__half *>(out_f16_dev), ld_out, static_cast<const unsigned *>(counters_dev),
                                  static_cast<unsigned long long *>(state_dev), sources, delta, err));
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}
