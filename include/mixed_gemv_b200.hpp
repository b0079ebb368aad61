// C++ face of libmixed_gemv_b200 with the reference's names, header-only over the C ABI
// (mixed_gemv_b200.h).  A maintainer of the reference's driver (mixed_gemv_test.cu) swaps
//     cutlass::gemm::device::GemvAdaptor<...>            -> mgv::GemvAdaptor<Bits, QuantOp>
//     host::utils::MixedGemvWeightPreprocessor::run      -> mgv::MixedGemvWeightPreprocessor::run  (device buffers)
//     host::utils::ZeroPointPreprocessor<...>::neg_...   -> mgv::ZeroPointPreprocessor::neg_zero_point_multiplies_scale
//     host::utils::SubBytePacker<...>::pack / unpack     -> mgv::SubBytePacker::pack / unpack
// and keeps the call sites: same member names, same argument order, same meaning.
//
// Naming: the reference calls the output-feature count M and the activation batch N
// (problem_size = {M, N, K} with N = 1 in its test); Arguments below keeps that order, the C ABI
// underneath uses N for features and M for the batch.
//
// Errors: the reference's adaptor prints a message and exits the process
// (gemv/device/gemv_adaptor.h:198-203, :236-252).  This adaptor prints the same kind of message
// and, by default, exits likewise; set exit_on_error = false to get the status back instead.
#pragma once

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "mixed_gemv_b200.h"

namespace mgv {

// cutlass::WeightOnlyQuantOp as used by the reference (gemv/warp/warp_dequantizer.h, mixed_gemv_test.cu:84-86)
enum class WeightOnlyQuantOp {
  UNDEFINED = MGV_QUANT_UNDEFINED,
  PER_COLUMN_SCALE_ONLY = MGV_QUANT_PER_COLUMN_SCALE_ONLY,
  FINEGRAINED_SCALE_ONLY = MGV_QUANT_FINEGRAINED_SCALE_ONLY,
  FINEGRAINED_SCALE_AND_ZEROS = MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS
};
// host::utils::QuantType and LayoutType (utils/preprocess.h)
enum class QuantType { W8_A16 = MGV_W8_A16, W4_A16 = MGV_W4_A16 };
enum class LayoutType { kRowMajor = MGV_LAYOUT_ROW_MAJOR, kColumnMajor = MGV_LAYOUT_COLUMN_MAJOR };

// cutlass::gemm::GemmCoord, as far as the adaptor's callers use it
struct GemmCoord {
  int m_, n_, k_;
  GemmCoord(int m = 0, int n = 0, int k = 0) : m_(m), n_(n), k_(k) {}
  int m() const { return m_; }
  int n() const { return n_; }
  int k() const { return k_; }
};
inline GemmCoord make_Coord(int m, int n, int k) { return GemmCoord(m, n, k); }

// cutlass::TensorRef: a pointer and a leading dimension (0 = "not given", as the reference's ldb)
template <class T>
struct TensorRef {
  T *ptr;
  long long stride;
  TensorRef(T *p = nullptr, long long s = 0) : ptr(p), stride(s) {}
  T *data() const { return ptr; }
};
template <class T>
TensorRef<T> make_TensorRef(T *p, long long stride) { return TensorRef<T>(p, stride); }

// EpilogueOutputOp::Params of LinearCombination: D = alpha * accumulator + beta * C
struct LinearCombinationParams {
  float alpha, beta;
  LinearCombinationParams(float a = 1.0f, float b = 1.0f) : alpha(a), beta(b) {}
};

inline mgv_status report(mgv_status st, const char *where, bool exit_on_error) {
  if (st != MGV_STATUS_OK) {
    std::fprintf(stderr, "%s: %s: %s\n", where, mgv_status_string(st), mgv_last_error());
    if (exit_on_error) std::exit(-1);
  }
  return st;
}

// cutlass::gemm::device::GemvAdaptor (gemv/device/gemv_adaptor.h:59-262).  The reference fixes
// the element types and the quantisation mode at compile time; so does this: Bits is 4 or 8,
// QuantOp the mode.  Every pointer is a device pointer.
template <int Bits, WeightOnlyQuantOp QuantOp>
class GemvAdaptor {
  static_assert(Bits == 4 || Bits == 8, "weights are 4 or 8 bits wide");

 public:
  using ElementA = void;        // preprocessed weights (opaque bytes)
  using ElementB = void;        // fp16 activations
  using ElementScale = void;    // fp16 scales / additive zeros
  using ElementC = void;        // fp16 bias and output

  struct Arguments {
    GemmCoord problem_size;                  // {M = output features, N = batch rows (1..16), K}
    TensorRef<ElementA const> ref_A;         // preprocessed weights (lda is implied by the layout)
    TensorRef<ElementB const> ref_B;         // x; stride 0 means K
    TensorRef<ElementScale const> ref_scale;
    TensorRef<ElementScale const> ref_zero_point;
    TensorRef<ElementC const> ref_C;         // bias, may be null
    TensorRef<ElementC> ref_D;               // output; stride 0 means M
    LinearCombinationParams epilogue;
    int group_size;
    int batch_count;
    long long batch_stride_A, batch_stride_B, batch_stride_scale, batch_stride_C, batch_stride_D;

    Arguments(GemmCoord problem_size_, TensorRef<ElementA const> ref_A_, TensorRef<ElementB const> ref_B_,
              TensorRef<ElementScale const> ref_scale_, TensorRef<ElementScale const> ref_zero_point_,
              TensorRef<ElementC const> ref_C_, TensorRef<ElementC> ref_D_,
              LinearCombinationParams epilogue_ = LinearCombinationParams(), int group_size_ = 64, int batch_count_ = 1,
              long long batch_stride_A_ = 0, long long batch_stride_B_ = 0, long long batch_stride_scale_ = 0,
              long long batch_stride_C_ = 0, long long batch_stride_D_ = 0)
        : problem_size(problem_size_), ref_A(ref_A_), ref_B(ref_B_), ref_scale(ref_scale_), ref_zero_point(ref_zero_point_),
          ref_C(ref_C_), ref_D(ref_D_), epilogue(epilogue_), group_size(group_size_), batch_count(batch_count_),
          batch_stride_A(batch_stride_A_), batch_stride_B(batch_stride_B_), batch_stride_scale(batch_stride_scale_),
          batch_stride_C(batch_stride_C_), batch_stride_D(batch_stride_D_) {}
  };

  bool exit_on_error = true;
  int variant = MGV_VARIANT_AUTO;  // MGV_VARIANT_SIMT keeps the reference's rounding points (batch <= 4)
  int flags = 0;                   // MGV_FLAG_*

  GemvAdaptor() { mgv_gemv_args_init(&args_); }
  ~GemvAdaptor() { mgv_gemv_plan_destroy(plan_); }
  GemvAdaptor(GemvAdaptor const &) = delete;
  GemvAdaptor &operator=(GemvAdaptor const &) = delete;

  // Validates the arguments and plans the launch once (the reference's initialize builds its
  // Params here, gemv_adaptor.h:198-223); run() then only launches.
  mgv_status initialize(Arguments const &a, mgv_stream_t = nullptr) {
    mgv_gemv_args_init(&args_);
    args_.N = a.problem_size.m();
    args_.M = a.problem_size.n();
    args_.K = a.problem_size.k();
    args_.weight_bits = Bits;
    args_.quant_op = int(QuantOp);
    args_.group_size = QuantOp == WeightOnlyQuantOp::PER_COLUMN_SCALE_ONLY ? a.problem_size.k() : a.group_size;
    args_.variant = variant;
    args_.flags = flags;
    args_.batch_count = a.batch_count;
    args_.weights = a.ref_A.data();
    args_.x = a.ref_B.data();
    args_.ldx = a.ref_B.stride ? a.ref_B.stride : a.problem_size.k();
    args_.scale = a.ref_scale.data();
    // the reference nulls the zero operand unless the mode has zeros (mixed_gemv_test.cu:145-147)
    args_.zero = QuantOp == WeightOnlyQuantOp::FINEGRAINED_SCALE_AND_ZEROS ? a.ref_zero_point.data() : nullptr;
    args_.bias = a.ref_C.data();
    args_.out = a.ref_D.data();
    args_.ldd = a.ref_D.stride ? a.ref_D.stride : a.problem_size.m();
    args_.alpha = a.epilogue.alpha;
    args_.beta = a.epilogue.beta;
    args_.batch_stride_weights = a.batch_stride_A;
    args_.batch_stride_x = a.batch_stride_B;
    args_.batch_stride_scale = a.batch_stride_scale;
    args_.batch_stride_bias = a.batch_stride_C;
    args_.batch_stride_out = a.batch_stride_D;
    return replan();
  }

  // Plans again from the C arguments: call it after changing them through c_args().
  mgv_status replan() {
    mgv_gemv_plan_destroy(plan_);
    plan_ = nullptr;
    return report(mgv_gemv_plan_create(&args_, &plan_), "Gemv adapter", exit_on_error);
  }

  // Enqueues the launch prepared by initialize() (gemv_adaptor.h:226-255).
  mgv_status run(mgv_stream_t stream = nullptr) {
    if (!plan_) return report(MGV_STATUS_INVALID_ARGUMENT, "Gemv adapter: run() before a successful initialize()", exit_on_error);
    return report(mgv_gemv_plan_run(plan_, stream), "Gemv adapter launch", exit_on_error);
  }

  mgv_status operator()(Arguments const &a, mgv_stream_t stream = nullptr) {
    const mgv_status st = initialize(a, stream);
    return st == MGV_STATUS_OK ? run(stream) : st;
  }

  // the C arguments, for callers that want to add what the reference has no word for
  // (workspace, peers, waits): change them after initialize(), then call replan()
  mgv_gemv_args &c_args() { return args_; }

 private:
  mgv_gemv_args args_;
  mgv_gemv_plan *plan_ = nullptr;
};

// host::utils::MixedGemvWeightPreprocessor::run (utils/preprocess.h:480-524), on device buffers:
// `quantized_weight` holds the un-preprocessed weights of logical shape `shape` ({K, N} or
// {experts, K, N}) in `layout`; the preprocessed bytes -- identical to the reference's -- land
// in `preprocessed_quantized_weight`.
struct MixedGemvWeightPreprocessor {
  static mgv_status run(void *preprocessed_quantized_weight, void const *quantized_weight, std::vector<size_t> const &shape,
                        LayoutType layout, QuantType quant_type, mgv_stream_t stream = nullptr, bool exit_on_error = true) {
    return report(mgv_preprocess_weights(preprocessed_quantized_weight, quantized_weight, shape.data(), int(shape.size()),
                                         int(layout), int(quant_type), stream),
                  "MixedGemvWeightPreprocessor", exit_on_error);
  }
};

// host::utils::ZeroPointPreprocessor::neg_zero_point_multiplies_scale (utils/preprocess.h:89-102)
struct ZeroPointPreprocessor {
  static mgv_status neg_zero_point_multiplies_scale(void *neg_zeros_x_scales, void const *scales, void const *zeros, size_t num_elts,
                                                    mgv_stream_t stream = nullptr, bool exit_on_error = true) {
    return report(mgv_preprocess_zeros(neg_zeros_x_scales, scales, zeros, num_elts, stream), "ZeroPointPreprocessor", exit_on_error);
  }
};

// host::utils::SubBytePacker<4, ...>::pack / unpack (utils/preprocess.h:22-86)
struct SubBytePacker {
  static mgv_status pack(void *packed_output, void const *unpacked_input, size_t num_elts, mgv_stream_t stream = nullptr,
                         bool exit_on_error = true) {
    return report(mgv_pack_int4(packed_output, unpacked_input, num_elts, stream), "SubBytePacker::pack", exit_on_error);
  }
  static mgv_status unpack(void *unpacked_output, void const *packed_input, size_t num_elts, mgv_stream_t stream = nullptr,
                           bool exit_on_error = true) {
    return report(mgv_unpack_int4(unpacked_output, packed_input, num_elts, stream), "SubBytePacker::unpack", exit_on_error);
  }
};

}  // namespace mgv
