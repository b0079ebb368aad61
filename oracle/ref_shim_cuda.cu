// Thin extern "C" shim over the reference's OWN CUDA kernel (its GemvAdaptor, instantiated with
// the configuration its test driver uses), compiled for sm_100a from the reference's headers
// where they lie (include paths come from oracle/Makefile; no reference source is copied).
// TEST AND BENCH INFRASTRUCTURE ONLY: a second checker for the device path (the reference's
// device arithmetic on the same buffers) and the "reference kernel recompiled for this GPU"
// figure that bench.py reports beside the library's.  Built against CUTLASS 4.5.0 headers
// (the reference pins 3.4.1, which is not available offline).
//
// The adaptor reports errors by printing and calling exit(-1); what it checks is checked here
// first and turned into a return code.
#include <cuda_runtime.h>

#include "cutlass/cutlass.h"
#include "cutlass/half.h"
#include "cutlass/array.h"
#include "cutlass/arch/mma.h"
#include "cutlass/arch/arch.h"
#include "cutlass/layout/matrix.h"
#include "cutlass/numeric_types.h"
#include "cutlass/epilogue/thread/activation.h"
#include "cutlass/gemm/kernel/default_gemm.h"
#include "cutlass/gemm/kernel/default_gemm_universal.h"
#include "cutlass/gemm/threadblock/threadblock_swizzle.h"
#include "cutlass/epilogue/thread/linear_combination.h"

#include "arch/mma.h"
#include "gemv/weight_only_quant_op.h"
#include "layout/tile_interleaved_layout.h"
#include "gemv/device/gemv_adaptor.h"

namespace {

using half_t = cutlass::half_t;
using WeightU4 = cutlass::uint4b_t;
constexpr int kAlignA = 128 / cutlass::sizeof_bits<WeightU4>::value;  // 32 weights per 128-bit access
constexpr int kAlignB = 128 / cutlass::sizeof_bits<half_t>::value;    // 8 activations
constexpr int kRows = kAlignA / kAlignB;                              // 4 interleaved rows
using LayoutA = cutlass::layout::RowMajorTileInterleave<kAlignB, kRows>;
using LayoutCol = cutlass::layout::ColumnMajor;
using OutputOp = cutlass::epilogue::thread::LinearCombination<half_t, kRows, float, float,
                                                             cutlass::epilogue::thread::ScaleType::OnlyAlphaScaling>;

// the driver's configuration (mixed_gemv_test.cu:30-112): SIMT, 64x1x64 block tile, 16x1x64 warp tile, one stage
template <cutlass::WeightOnlyQuantOp Op>
using Adaptor = cutlass::gemm::device::GemvAdaptor<
    WeightU4, LayoutA, half_t, LayoutCol, half_t, LayoutCol, half_t, LayoutCol, float, cutlass::arch::OpClassSimt,
    cutlass::arch::Sm50, typename cutlass::arch::TagOperator<cutlass::arch::OpMultiplyAdd, Op>::TaggedOperator,
    cutlass::gemm::GemmShape<64, 1, 64>, cutlass::gemm::GemmShape<16, 1, 64>, cutlass::gemm::GemmShape<1, 1, 1>,
    cutlass::MatrixShape<4, 8>, OutputOp, 1, kAlignA, kAlignB, kRows>;

template <cutlass::WeightOnlyQuantOp Op>
int run(const void *A, const void *B, const void *scale, const void *zero, void *D, int features, int K, int group,
        cudaStream_t stream) {
  using Dev = Adaptor<Op>;
  // device_gemv(), mixed_gemv_test.cu:124-165: lda = 4K, ldb = 0, scale stride = features, C = null
  typename Dev::Arguments args{cutlass::make_Coord(features, 1, K),
                               {reinterpret_cast<WeightU4 *>(const_cast<void *>(A)), K * LayoutA::kRowsInterleaved},
                               cutlass::make_TensorRef(static_cast<const half_t *>(B), LayoutCol(0)),
                               cutlass::make_TensorRef(static_cast<const half_t *>(scale), LayoutCol(features)),
                               cutlass::make_TensorRef(static_cast<const half_t *>(zero), LayoutCol(features)),
                               {nullptr, features},
                               cutlass::make_TensorRef(static_cast<half_t *>(D), LayoutCol(features)),
                               {},
                               group};
  Dev op;
  op.initialize(args);
  op.run(stream);
  return 0;
}

}  // namespace

// quant_op: 2 = FINEGRAINED_SCALE_ONLY, 3 = FINEGRAINED_SCALE_AND_ZEROS (4-bit weights, one activation row).
// Returns 0, or -1 for what the reference cannot run (it would exit): groups other than 64 / 128
// (its scale pointer only steps for those), shapes off its tiling.
extern "C" int ref_device_gemv(int quant_op, const void *weights_preprocessed, const void *x, const void *scale,
                               const void *zero, void *out, int features, int K, int group, void *stream) {
  if (!weights_preprocessed || !x || !scale || !out) return -1;
  if (group != 64 && group != 128) return -1;
  if (features % 4 || K % 64 || K % group) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (quant_op == 2) return run<cutlass::WeightOnlyQuantOp::FINEGRAINED_SCALE_ONLY>(weights_preprocessed, x, scale, nullptr, out, features, K, group, s);
  if (quant_op == 3 && zero)
    return run<cutlass::WeightOnlyQuantOp::FINEGRAINED_SCALE_AND_ZEROS>(weights_preprocessed, x, scale, zero, out, features, K, group, s);
  return -1;
}
