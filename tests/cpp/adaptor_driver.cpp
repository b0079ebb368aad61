// Drives the C++ face (mixed_gemv_b200.hpp) the way the reference's mixed_gemv_test.cu drives
// its adaptor: preprocess the weights, preprocess the zero-points, device_gemv().  Input and
// output travel in flat binary files written and read by tests/test_gpu_cpp_mirror.py.
//
// input:  int32 header {features M, batch N, K, bits, quant_op, group_size, has_bias, 0}
//         raw weights (column-major, packed for 4 bits), x fp16 [N][K], scale fp16 [G][M],
//         zero-points int8 [G][M] (mode 3 only), bias fp16 [M] (if has_bias)
// output: fp16 [N][M]
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <vector>

#include "mixed_gemv_b200.hpp"

#define CK(x)                                                                      \
  do {                                                                             \
    cudaError_t e__ = (x);                                                         \
    if (e__ != cudaSuccess) {                                                      \
      std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e__));               \
      return 2;                                                                    \
    }                                                                              \
  } while (0)

template <int Bits, mgv::WeightOnlyQuantOp Op>
int device_gemv(const void *A, const void *B, const void *scale, const void *zero, const void *C, void *D, int M, int N, int K,
                int group_size) {
  using DeviceKernel = mgv::GemvAdaptor<Bits, Op>;
  typename DeviceKernel::Arguments args{mgv::make_Coord(M, N, K),
                                        {A, 0},
                                        mgv::make_TensorRef(B, 0),
                                        mgv::make_TensorRef(scale, M),
                                        mgv::make_TensorRef(zero, M),
                                        {C, M},
                                        mgv::make_TensorRef(D, M),
                                        {},
                                        group_size};
  DeviceKernel op;
  op.initialize(args);
  op.run();
  return 0;
}

int main(int argc, char **argv) {
  if (argc != 3) return 1;
  FILE *f = std::fopen(argv[1], "rb");
  if (!f) return 1;
  int32_t h[8];
  if (std::fread(h, 4, 8, f) != 8) return 1;
  const int M = h[0], N = h[1], K = h[2], bits = h[3], op = h[4], group = h[5], has_bias = h[6];
  const int G = op == 1 ? 1 : K / group;
  const size_t w_bytes = size_t(M) * K * bits / 8, x_bytes = size_t(N) * K * 2, s_bytes = size_t(G) * M * 2;
  std::vector<uint8_t> w(w_bytes), x(x_bytes), s(s_bytes), z(op == 3 ? size_t(G) * M : 0), b(has_bias ? size_t(M) * 2 : 0);
  if (std::fread(w.data(), 1, w_bytes, f) != w_bytes || std::fread(x.data(), 1, x_bytes, f) != x_bytes ||
      std::fread(s.data(), 1, s_bytes, f) != s_bytes || std::fread(z.data(), 1, z.size(), f) != z.size() ||
      std::fread(b.data(), 1, b.size(), f) != b.size())
    return 1;
  std::fclose(f);

  void *d_raw, *d_A, *d_B, *d_scale, *d_zi8 = nullptr, *d_zero = nullptr, *d_C = nullptr, *d_D;
  CK(cudaMalloc(&d_raw, w_bytes));
  CK(cudaMalloc(&d_A, w_bytes));
  CK(cudaMalloc(&d_B, x_bytes));
  CK(cudaMalloc(&d_scale, s_bytes));
  CK(cudaMalloc(&d_D, size_t(N) * M * 2));
  CK(cudaMemcpy(d_raw, w.data(), w_bytes, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_B, x.data(), x_bytes, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_scale, s.data(), s_bytes, cudaMemcpyHostToDevice));
  if (op == 3) {
    CK(cudaMalloc(&d_zi8, z.size()));
    CK(cudaMalloc(&d_zero, s_bytes));
    CK(cudaMemcpy(d_zi8, z.data(), z.size(), cudaMemcpyHostToDevice));
    // mixed_gemv_test.cu:236-239
    mgv::ZeroPointPreprocessor::neg_zero_point_multiplies_scale(d_zero, d_scale, d_zi8, size_t(G) * M);
  }
  if (has_bias) {
    CK(cudaMalloc(&d_C, size_t(M) * 2));
    CK(cudaMemcpy(d_C, b.data(), size_t(M) * 2, cudaMemcpyHostToDevice));
  }
  // mixed_gemv_test.cu:245-254
  mgv::MixedGemvWeightPreprocessor::run(d_A, d_raw, {size_t(K), size_t(M)}, mgv::LayoutType::kColumnMajor,
                                        bits == 4 ? mgv::QuantType::W4_A16 : mgv::QuantType::W8_A16);
  using Op = mgv::WeightOnlyQuantOp;
  int rc = 3;
  if (bits == 4 && op == 3) rc = device_gemv<4, Op::FINEGRAINED_SCALE_AND_ZEROS>(d_A, d_B, d_scale, d_zero, d_C, d_D, M, N, K, group);
  if (bits == 4 && op == 2) rc = device_gemv<4, Op::FINEGRAINED_SCALE_ONLY>(d_A, d_B, d_scale, nullptr, d_C, d_D, M, N, K, group);
  if (bits == 8 && op == 1) rc = device_gemv<8, Op::PER_COLUMN_SCALE_ONLY>(d_A, d_B, d_scale, nullptr, d_C, d_D, M, N, K, group);
  if (rc) return rc;
  CK(cudaDeviceSynchronize());
  std::vector<uint8_t> out(size_t(N) * M * 2);
  CK(cudaMemcpy(out.data(), d_D, out.size(), cudaMemcpyDeviceToHost));
  f = std::fopen(argv[2], "wb");
  if (!f || std::fwrite(out.data(), 1, out.size(), f) != out.size()) return 1;
  std::fclose(f);

  // error behaviour: a refused call reports instead of exiting when asked to
  mgv::GemvAdaptor<4, Op::FINEGRAINED_SCALE_ONLY> bad;
  bad.exit_on_error = false;
  mgv::GemvAdaptor<4, Op::FINEGRAINED_SCALE_ONLY>::Arguments ba{mgv::make_Coord(M, 17, K), {d_A, 0}, {d_B, 0}, {d_scale, M}, {nullptr, M},
                                                                {nullptr, M}, {d_D, M}, {}, group};
  if (bad.initialize(ba) == MGV_STATUS_OK || bad.run() == MGV_STATUS_OK) return 4;  // a batch of 17 is refused
  std::puts("ok");
  return 0;
}
