// Memory windows and arrival counters for the output exchange of an N-split (sharded) layer.
//
// The reference is single-GPU.  When one layer is cut over the GPUs of a node along its output
// features, every GPU needs every other GPU's slice of the output before the next layer.  Here
// the GEMV's epilogue stores each output element straight into all GPUs' gather buffers (peer
// stores over NVLink) and counts its thread blocks in on a per-GPU arrival counter, so the
// exchange overlaps the kernel's tail and needs no collective call; what is left for the
// consumer is a bounded wait on its own counter.  This file holds the host plumbing: windows
// that other processes can map (CUDA IPC) and the wait.
#include <cstring>

#include "mgv_common.cuh"

namespace mgv {

// One thread polls the counter with system-scope acquire loads until it has grown by `delta`
// beyond *seen, then moves *seen on.  The wait is bounded by the global timer: a peer that never
// arrives costs about a second, raises the error word and lets the stream continue.
__global__ void wait_arrivals_kernel(const unsigned *flag, unsigned *seen, unsigned delta, int *error_word) {
  const unsigned target = *seen + delta;
  *seen = target;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (int(v - target) >= 0) return;
    }
    if (global_timer_ns() - t0 > 1000000000ull) {
      atomicOr(error_word, 0x20);
      return;
    }
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

extern "C" mgv_status mgv_wait_arrivals(const void *flag_dev, void *seen_dev, uint32_t delta, mgv_stream_t s) {
  if (!flag_dev || !seen_dev) return fail(MGV_STATUS_INVALID_ARGUMENT, "wait_arrivals: null counter");
  if (reinterpret_cast<uintptr_t>(flag_dev) % 4 || reinterpret_cast<uintptr_t>(seen_dev) % 4)
    return fail(MGV_STATUS_MISALIGNED, "wait_arrivals: the counters must be 4-byte aligned");
  int *err = device_error_word();
  if (!err) return fail(MGV_STATUS_CUDA_ERROR, "wait_arrivals: no device error word");
  wait_arrivals_kernel<<<1, 1, 0, static_cast<cudaStream_t>(s)>>>(static_cast<const unsigned *>(flag_dev),
                                                                  static_cast<unsigned *>(seen_dev), delta, err);
  MGV_CUDA_TRY(cudaGetLastError());
  return MGV_STATUS_OK;
}
