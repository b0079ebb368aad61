// Status plumbing and the resident-layer handle of the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "mgv_common.cuh"

namespace mgv {

static thread_local char tl_error[512] = "";

mgv_status fail(mgv_status st, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return st;
}

mgv_status cuda_fail(cudaError_t err, const char *what) {
  snprintf(tl_error, sizeof(tl_error), "%s: %s", what, cudaGetErrorString(err));
  return MGV_STATUS_CUDA_ERROR;
}

}  // namespace mgv

namespace mgv {

// Brings x from mapped pinned host memory into device memory (one block: 8 KB to 128 KB over
// PCIe).  It lets the next kernel of the stream start at once (programmatic dependent launch):
// the GEMV behind it prefetches its weights while x is still on the bus, and waits for this
// kernel only before it reads x.
__global__ void upload_x_kernel(uint4 *dst, const uint4 *src_host, size_t n16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (size_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src_host[i];
}

}  // namespace mgv

using namespace mgv;

extern "C" const char *mgv_status_string(int st) {
  switch (st) {
    case MGV_STATUS_OK: return "ok";
    case MGV_STATUS_INVALID_ARGUMENT: return "invalid argument";
    case MGV_STATUS_UNSUPPORTED: return "unsupported";
    case MGV_STATUS_MISALIGNED: return "misaligned";
    case MGV_STATUS_WORKSPACE_TOO_SMALL: return "workspace too small";
    case MGV_STATUS_CUDA_ERROR: return "CUDA error";
    case MGV_STATUS_DEVICE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

extern "C" const char *mgv_last_error(void) { return tl_error; }

extern "C" int mgv_version(void) { return 100; }

// ---- resident layer -------------------------------------------------------------------------

struct mgv_linear {
  int N = 0, K = 0, bits = 0, quant_op = 0, group = 0, max_M = 0, device = 0;
  void *w = nullptr, *scale = nullptr, *zero = nullptr, *bias = nullptr;
  void *x = nullptr, *out = nullptr, *ws = nullptr;
  size_t ws_bytes = 0;
  cudaStream_t stream = nullptr;
  // forward_host with pinned buffers replays a two-node graph (x upload, GEMV writing straight
  // into the mapped host buffer); rebuilt when the buffers, M or the variant change
  cudaGraphExec_t host_exec = nullptr;
  const void *host_x = nullptr;
  void *host_out = nullptr;
  int host_M = 0, host_variant = 0;
  bool warmed = false;
};

static void release(mgv_linear *l) {
  if (!l) return;
  if (l->host_exec) cudaGraphExecDestroy(l->host_exec);
  cudaFree(l->w); cudaFree(l->scale); cudaFree(l->zero); cudaFree(l->bias);
  cudaFree(l->x); cudaFree(l->out); cudaFree(l->ws);
  if (l->stream) cudaStreamDestroy(l->stream);
  delete l;
}

#define MGV_TRY_L(expr)                                          \
  do {                                                           \
    cudaError_t e__ = (expr);                                    \
    if (e__ != cudaSuccess) { release(l); return cuda_fail(e__, #expr); } \
  } while (0)

static void fill_args(const mgv_linear *l, mgv_gemv_args *a, const void *x, void *out, int M, int variant, int flags = 0) {
  mgv_gemv_args_init(a);
  a->flags = flags;
  a->M = M; a->N = l->N; a->K = l->K;
  a->weight_bits = l->bits; a->quant_op = l->quant_op; a->group_size = l->group;
  a->variant = variant;
  a->weights = l->w; a->x = x; a->ldx = l->K; a->scale = l->scale; a->zero = l->zero; a->bias = l->bias;
  a->out = out; a->ldd = l->N;
  a->workspace = l->ws; a->workspace_bytes = l->ws_bytes;
}

extern "C" mgv_status mgv_linear_create(mgv_linear **out, int N, int K, int bits, int quant_op, int group_size,
                                        int layout, const void *w_host, const void *scale_host,
                                        const void *zeros_host, const void *bias_host, int max_M) {
  if (!out) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_create: null handle pointer");
  *out = nullptr;
  if (!w_host || !scale_host) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_create: null weights or scales");
  if (bits != 4 && bits != 8) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_create: weight_bits must be 4 or 8");
  if (max_M < 1 || max_M > 16) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_create: max_M must be 1..16");
  if (N < 1 || K < 1) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_create: bad shape");
  if (quant_op == MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS && !zeros_host)
    return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_create: the mode needs zeros");
  mgv_linear *l = new (std::nothrow) mgv_linear;
  if (!l) return fail(MGV_STATUS_CUDA_ERROR, "linear_create: out of host memory");
  l->N = N; l->K = K; l->bits = bits; l->quant_op = quant_op; l->max_M = max_M;
  l->group = quant_op == MGV_QUANT_PER_COLUMN_SCALE_ONLY ? K : group_size;
  if (l->group < 1 || K % l->group) { release(l); return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_create: K %% group_size != 0"); }
  const size_t w_bytes = size_t(N) * K * bits / 8;
  const size_t sg_bytes = size_t(K / l->group) * N * 2;
  MGV_TRY_L(cudaGetDevice(&l->device));
  MGV_TRY_L(cudaStreamCreateWithFlags(&l->stream, cudaStreamNonBlocking));
  void *raw = nullptr;
  MGV_TRY_L(cudaMalloc(&l->w, w_bytes));
  MGV_TRY_L(cudaMalloc(&raw, w_bytes));
  cudaError_t e = cudaMemcpyAsync(raw, w_host, w_bytes, cudaMemcpyHostToDevice, l->stream);
  if (e != cudaSuccess) { cudaFree(raw); release(l); return cuda_fail(e, "weight upload"); }
  const size_t shape[2] = {size_t(K), size_t(N)};
  mgv_status st = mgv_preprocess_weights(l->w, raw, shape, 2, layout, bits == 4 ? MGV_W4_A16 : MGV_W8_A16, l->stream);
  e = cudaStreamSynchronize(l->stream);
  cudaFree(raw);
  if (st != MGV_STATUS_OK) { release(l); return st; }
  if (e != cudaSuccess) { release(l); return cuda_fail(e, "weight preprocessing"); }
  MGV_TRY_L(cudaMalloc(&l->scale, sg_bytes));
  MGV_TRY_L(cudaMemcpy(l->scale, scale_host, sg_bytes, cudaMemcpyHostToDevice));
  if (quant_op == MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS) {
    MGV_TRY_L(cudaMalloc(&l->zero, sg_bytes));
    MGV_TRY_L(cudaMemcpy(l->zero, zeros_host, sg_bytes, cudaMemcpyHostToDevice));
  }
  if (bias_host) {
    MGV_TRY_L(cudaMalloc(&l->bias, size_t(N) * 2));
    MGV_TRY_L(cudaMemcpy(l->bias, bias_host, size_t(N) * 2, cudaMemcpyHostToDevice));
  }
  MGV_TRY_L(cudaMalloc(&l->x, size_t(max_M) * K * 2));
  MGV_TRY_L(cudaMalloc(&l->out, size_t(max_M) * N * 2));
  mgv_gemv_args a;
  fill_args(l, &a, l->x, l->out, max_M, MGV_VARIANT_AUTO);
  st = mgv_gemv_workspace_size(&a, &l->ws_bytes);
  if (st != MGV_STATUS_OK) { release(l); return st; }
  if (l->ws_bytes) {
    MGV_TRY_L(cudaMalloc(&l->ws, l->ws_bytes));
    MGV_TRY_L(cudaMemset(l->ws, 0, l->ws_bytes));
  }
  *out = l;
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_linear_forward(mgv_linear *l, const void *x_dev, void *out_dev, int M, int variant,
                                         mgv_stream_t s) {
  if (!l || !x_dev || !out_dev) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_forward: null argument");
  if (M < 1 || M > l->max_M) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_forward: M=%d outside 1..%d", M, l->max_M);
  mgv_gemv_args a;
  fill_args(l, &a, x_dev, out_dev, M, variant);
  return mgv_gemv(&a, s);
}

// Device address of a pinned, mapped host buffer, or null when the buffer is pageable.
static void *mapped_device_pointer(const void *host) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, host) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return at.type == cudaMemoryTypeHost ? at.devicePointer : nullptr;
}

static mgv_status forward_host_copies(mgv_linear *l, const void *x_host, void *out_host, int M, int variant) {
  MGV_CUDA_TRY(cudaMemcpyAsync(l->x, x_host, size_t(M) * l->K * 2, cudaMemcpyHostToDevice, l->stream));
  mgv_status st = mgv_linear_forward(l, l->x, l->out, M, variant, l->stream);
  if (st != MGV_STATUS_OK) return st;
  MGV_CUDA_TRY(cudaMemcpyAsync(out_host, l->out, size_t(M) * l->N * 2, cudaMemcpyDeviceToHost, l->stream));
  MGV_CUDA_TRY(cudaStreamSynchronize(l->stream));
  return MGV_STATUS_OK;
}

extern "C" mgv_status mgv_linear_forward_host(mgv_linear *l, const void *x_host, void *out_host, int M, int variant) {
  if (!l || !x_host || !out_host) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_forward_host: null argument");
  if (M < 1 || M > l->max_M) return fail(MGV_STATUS_INVALID_ARGUMENT, "linear_forward_host: M=%d outside 1..%d", M, l->max_M);
  // The first call runs the plain sequence (it also sets the kernels' attributes, which a stream
  // capture must not do); so does every call with pageable buffers.
  void *out_dev = mapped_device_pointer(out_host);
  const void *x_dev = mapped_device_pointer(x_host);
  if (!l->warmed || !out_dev || !x_dev || (size_t(M) * l->K * 2) % 16 || reinterpret_cast<uintptr_t>(x_dev) % 16) {
    mgv_status st = forward_host_copies(l, x_host, out_host, M, variant);
    if (st == MGV_STATUS_OK) l->warmed = true;
    return st;
  }
  // Pinned buffers: one graph launch per call -- a one-block kernel that reads x over PCIe, and a
  // GEMV (dependent launch: it prefetches weights meanwhile) whose epilogue writes the result over
  // PCIe straight into the caller's buffer (posted writes: no read-back copy).
  if (!l->host_exec || l->host_x != x_host || l->host_out != out_host || l->host_M != M || l->host_variant != variant) {
    if (l->host_exec) {
      cudaGraphExecDestroy(l->host_exec);
      l->host_exec = nullptr;
    }
    cudaGraph_t graph = nullptr;
    MGV_CUDA_TRY(cudaStreamBeginCapture(l->stream, cudaStreamCaptureModeThreadLocal));
    upload_x_kernel<<<1, 512, 0, l->stream>>>(static_cast<uint4 *>(l->x), static_cast<const uint4 *>(x_dev), size_t(M) * l->K * 2 / 16);
    cudaError_t e = cudaGetLastError();
    mgv_status st = MGV_STATUS_CUDA_ERROR;
    if (e == cudaSuccess) {
      mgv_gemv_args a;
      fill_args(l, &a, l->x, out_dev, M, variant, MGV_FLAG_PDL);  // starts while x is still on the bus
      st = mgv_gemv(&a, l->stream);
    }
    const cudaError_t e2 = cudaStreamEndCapture(l->stream, &graph);
    if (e != cudaSuccess || st != MGV_STATUS_OK || e2 != cudaSuccess || !graph) {
      if (graph) cudaGraphDestroy(graph);
      (void)cudaGetLastError();
      return forward_host_copies(l, x_host, out_host, M, variant);  // capture refused: the plain sequence still serves
    }
    e = cudaGraphInstantiate(&l->host_exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
      l->host_exec = nullptr;
      (void)cudaGetLastError();
      return forward_host_copies(l, x_host, out_host, M, variant);
    }
    l->host_x = x_host; l->host_out = out_host; l->host_M = M; l->host_variant = variant;
  }
  MGV_CUDA_TRY(cudaGraphLaunch(l->host_exec, l->stream));
  MGV_CUDA_TRY(cudaStreamSynchronize(l->stream));
  return MGV_STATUS_OK;
}

extern "C" const void *mgv_linear_weights(const mgv_linear *l) { return l ? l->w : nullptr; }

extern "C" void mgv_linear_destroy(mgv_linear *l) { release(l); }
