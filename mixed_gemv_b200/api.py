"""Host-side mirror of the reference's interface for this path, over the C ABI.

Same names, argument meaning and order as the reference's C++ entry points; tensors are
torch CUDA tensors whose ``data_ptr()`` crosses the ABI.  Where the reference prints and
calls ``exit(-1)`` these raise :class:`MgvError` carrying the library's status.

    SubBytePacker                      utils/preprocess.h:24-85
    ZeroPointPreprocessor              utils/preprocess.h:88-102
    MixedGemvWeightPreprocessor.run    utils/preprocess.h:480-522
    GemvAdaptor / Arguments            gemv/device/gemv_adaptor.h:59-262
    device_gemv                        mixed_gemv_test.cu:124-165
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import GemvArgs, LaunchInfo, MgvError, check
from .enums import LayoutType, QuantType, Variant, WeightOnlyQuantOp


def _stream_ptr(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def _dev_ptr(t: Optional[torch.Tensor], name: str) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise MgvError(1, f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise MgvError(1, f"{name} must be contiguous")
    return t.data_ptr()


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("mixed_gemv_b200 needs a CUDA device; there is no CPU fallback")
    _lib.load()


class SubBytePacker:
    """SubBytePacker<int4b_t, int8_t> (utils/preprocess.h:24-85) on the GPU."""

    @staticmethod
    def pack(packed_output: torch.Tensor, unpacked_input: torch.Tensor, unpacked_num_elements: int,
             stream=None) -> None:
        check(_lib.load().mgv_pack_int4(_dev_ptr(packed_output, "packed_output"),
                                        _dev_ptr(unpacked_input, "unpacked_input"),
                                        int(unpacked_num_elements), _stream_ptr(stream)))

    @staticmethod
    def unpack(unpacked_output: torch.Tensor, packed_input: torch.Tensor, packed_num_elements: int,
               stream=None) -> None:
        check(_lib.load().mgv_unpack_int4(_dev_ptr(unpacked_output, "unpacked_output"),
                                          _dev_ptr(packed_input, "packed_input"),
                                          int(packed_num_elements), _stream_ptr(stream)))


class ZeroPointPreprocessor:
    """ZeroPointPreprocessor<half, int8_t> (utils/preprocess.h:88-102) on the GPU."""

    @staticmethod
    def neg_zero_point_multiplies_scale(neg_zeros_x_scales: torch.Tensor, scales: torch.Tensor,
                                        zeros: torch.Tensor, n: int, stream=None) -> None:
        check(_lib.load().mgv_preprocess_zeros(_dev_ptr(neg_zeros_x_scales, "neg_zeros_x_scales"),
                                               _dev_ptr(scales, "scales"), _dev_ptr(zeros, "zeros"),
                                               int(n), _stream_ptr(stream)))


class MixedGemvWeightPreprocessor:
    """MixedGemvWeightPreprocessor (utils/preprocess.h:480-522) on the GPU, bit-exact."""

    @staticmethod
    def run(preprocessed_quantized_weight: torch.Tensor, quantized_weight: torch.Tensor,
            shape: Sequence[int], weight_layout: LayoutType, quant_type: QuantType,
            force_interleave: bool = False, stream=None) -> None:
        # force_interleave is accepted and ignored, as in the reference (:484).
        arr = (C.c_size_t * len(shape))(*[int(s) for s in shape])
        check(_lib.load().mgv_preprocess_weights(
            _dev_ptr(preprocessed_quantized_weight, "preprocessed_quantized_weight"),
            _dev_ptr(quantized_weight, "quantized_weight"), arr, len(shape), int(weight_layout),
            int(quant_type), _stream_ptr(stream)))


@dataclass
class Arguments:
    """GemvAdaptor::Arguments (gemv/device/gemv_adaptor.h:114-178) in this library's naming:
    problem (N, M, K) with N output features; ref_A = weights (preprocessed), ref_B = x,
    ref_C = bias (epilogue source, may be None), ref_D = out."""
    M: int
    N: int
    K: int
    weights: torch.Tensor
    x: torch.Tensor
    scale: torch.Tensor
    out: torch.Tensor
    zero: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None
    weight_bits: int = 4
    quant_op: WeightOnlyQuantOp = WeightOnlyQuantOp.FINEGRAINED_SCALE_ONLY
    group_size: int = 64
    alpha: float = 1.0
    beta: float = 1.0
    batch_count: int = 1
    batch_stride_weights: int = 0
    batch_stride_x: int = 0
    batch_stride_scale: int = 0
    batch_stride_bias: int = 0
    batch_stride_out: int = 0
    ldx: Optional[int] = None
    ldd: Optional[int] = None
    variant: Variant = Variant.AUTO
    flags: int = 0
    hints: int = 0                       # _lib.HINT_*: forces a code path (tests, tuning)
    workspace: Optional[torch.Tensor] = None
    # fused output exchange of an N-split layer: device addresses (ints) of the peers' output
    # buffers and arrival counters, see mixed_gemv_b200.exchange
    peer_out: tuple = ()
    peer_flag: tuple = ()
    # consumer side inside the kernel: device addresses of this GPU's per-source arrival counters
    # and of the 8-byte launch counter, the arrivals one launch of one source brings, and the mask
    # of the sources waited for
    wait_flag: int = 0
    wait_state: int = 0
    wait_delta: int = 0
    wait_sources: int = 0
    # prefetch hint: a tensor a later call will read (normally the next layer's weights)
    prefetch: Optional[torch.Tensor] = None


class GemvAdaptor:
    """GemvAdaptor (gemv/device/gemv_adaptor.h:59-262): initialize() validates the arguments and
    plans the launch once (mgv_gemv_plan_create), run() only launches (mgv_gemv_plan_run), calling
    the object does both."""

    def __init__(self):
        self._args: Optional[GemvArgs] = None
        self._keep = None
        self._plan = None

    def _drop_plan(self):
        if getattr(self, "_plan", None):
            _lib.load().mgv_gemv_plan_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self._drop_plan()
        except Exception:
            pass

    @staticmethod
    def _to_c(a: Arguments) -> GemvArgs:
        lib = _lib.load()
        c = GemvArgs()
        lib.mgv_gemv_args_init(C.byref(c))
        c.M, c.N, c.K = int(a.M), int(a.N), int(a.K)
        c.weight_bits, c.quant_op, c.group_size = int(a.weight_bits), int(a.quant_op), int(a.group_size)
        c.variant, c.flags, c.batch_count = int(a.variant), int(a.flags), int(a.batch_count)
        c.hints = int(a.hints)
        c.weights = _dev_ptr(a.weights, "weights")
        c.x = _dev_ptr(a.x, "x")
        c.scale = _dev_ptr(a.scale, "scale")
        # the reference nulls the zero operand unless the mode has zeros (mixed_gemv_test.cu:145-147)
        has_zero = WeightOnlyQuantOp(a.quant_op) == WeightOnlyQuantOp.FINEGRAINED_SCALE_AND_ZEROS
        c.zero = _dev_ptr(a.zero, "zero") if has_zero else None
        c.bias = _dev_ptr(a.bias, "bias")
        c.out = _dev_ptr(a.out, "out")
        c.ldx = int(a.ldx if a.ldx is not None else a.K)
        c.ldd = int(a.ldd if a.ldd is not None else a.N)
        c.alpha, c.beta = float(a.alpha), float(a.beta)
        c.batch_stride_weights = int(a.batch_stride_weights)
        c.batch_stride_x = int(a.batch_stride_x)
        c.batch_stride_scale = int(a.batch_stride_scale)
        c.batch_stride_bias = int(a.batch_stride_bias)
        c.batch_stride_out = int(a.batch_stride_out)
        if a.workspace is not None:
            c.workspace = _dev_ptr(a.workspace, "workspace")
            c.workspace_bytes = a.workspace.numel() * a.workspace.element_size()
        if len(a.peer_out) > 8 or (a.peer_flag and len(a.peer_flag) != len(a.peer_out)):
            raise MgvError(1, "peer_out holds at most 8 addresses and peer_flag one per peer_out")
        c.n_peers = len(a.peer_out)
        for i, ptr in enumerate(a.peer_out):
            c.peer_out[i] = int(ptr)
            c.peer_flag[i] = int(a.peer_flag[i]) if a.peer_flag and a.peer_flag[i] else None
        if a.wait_flag:
            c.wait_flag, c.wait_state, c.wait_delta = int(a.wait_flag), int(a.wait_state), int(a.wait_delta)
            c.wait_sources = int(a.wait_sources)
        if a.prefetch is not None:
            c.prefetch = _dev_ptr(a.prefetch, "prefetch")
            c.prefetch_bytes = a.prefetch.numel() * a.prefetch.element_size()
        return c

    @staticmethod
    def get_workspace_size(args: Arguments) -> int:
        c = GemvAdaptor._to_c(args)
        n = C.c_size_t(0)
        check(_lib.load().mgv_gemv_workspace_size(C.byref(c), C.byref(n)))
        return int(n.value)

    @staticmethod
    def allocate_workspace(args: Arguments) -> Optional[torch.Tensor]:
        """Zeroed split-K scratch for these arguments, or None when the shape needs none."""
        n = GemvAdaptor.get_workspace_size(args)
        if n == 0:
            return None
        return torch.zeros(n, dtype=torch.uint8, device=args.weights.device)

    def initialize(self, args: Arguments, stream=None) -> None:
        c = self._to_c(args)
        info = LaunchInfo()
        lib = _lib.load()
        check(lib.mgv_gemv_launch_info(C.byref(c), C.byref(info)))
        self._drop_plan()
        plan = C.c_void_p()
        check(lib.mgv_gemv_plan_create(C.byref(c), C.byref(plan)))
        self._args, self._keep, self.launch_info, self._plan = c, args, info, plan

    def run(self, stream=None) -> None:
        if self._plan is None:
            raise MgvError(1, "GemvAdaptor.run() before initialize()")
        check(_lib.load().mgv_gemv_plan_run(self._plan, _stream_ptr(stream)))

    def run_static_scratch(self, stream=None) -> None:
        """run() through mgv_gemv_static_scratch: for callers that may not allocate device memory
        (stream capture in progress, plug-ins with a fixed memory budget).  Any workspace in the
        arguments is ignored; the library's built-in 4 MiB scratch array is used instead."""
        if self._args is None:
            raise MgvError(1, "GemvAdaptor.run_static_scratch() before initialize()")
        check(_lib.load().mgv_gemv_static_scratch(C.byref(self._args), _stream_ptr(stream)))

    def __call__(self, args: Arguments, stream=None) -> None:
        self.initialize(args, stream)
        self.run(stream)


def device_gemv(ptr_A: torch.Tensor, ptr_B: torch.Tensor, ptr_scale: torch.Tensor,
                ptr_zero_point: Optional[torch.Tensor], ptr_C: Optional[torch.Tensor],
                ptr_D: torch.Tensor, B: int, M: int, N: int, K: int, group_size: int, *,
                quant_op: WeightOnlyQuantOp = WeightOnlyQuantOp.FINEGRAINED_SCALE_AND_ZEROS,
                weight_bits: int = 4, variant: Variant = Variant.AUTO,
                workspace: Optional[torch.Tensor] = None, stream=None) -> None:
    """device_gemv (mixed_gemv_test.cu:124-165) with the reference's argument order and naming:
    here ``M`` is the number of OUTPUT FEATURES and ``N`` the number of activation rows (the
    reference fixes it to 1), ``B`` the batch count.  The quantisation mode, a compile-time
    constant in the reference (:84-86), is a keyword."""
    args = Arguments(M=N, N=M, K=K, weights=ptr_A, x=ptr_B, scale=ptr_scale, zero=ptr_zero_point,
                     bias=ptr_C, out=ptr_D, weight_bits=weight_bits, quant_op=quant_op,
                     group_size=group_size, batch_count=B, variant=variant, workspace=workspace)
    op = GemvAdaptor()
    op.initialize(args, stream)
    op.run(stream)


def device_error_state() -> int:
    """0, or the code a bounded device-side wait left when it gave up (synchronises)."""
    v = C.c_int(0)
    st = _lib.load().mgv_device_error_state(C.byref(v))
    if st not in (0, 6):
        check(st)
    return int(v.value)


class Linear:
    """A resident quantised layer behind one handle (mgv_linear_*): uploads and preprocesses
    host weights once, then serves host-buffer or device-buffer forwards -- the flow of
    main() in mixed_gemv_test.cu:245-283."""

    def __init__(self, case_or_none=None, *, N=None, K=None, weight_bits=4,
                 quant_op=WeightOnlyQuantOp.FINEGRAINED_SCALE_ONLY, group_size=128,
                 layout=LayoutType.kColumnMajor, weights=None, scale=None, zeros=None, bias=None,
                 max_M=1):
        import numpy as np
        require_cuda()
        if case_or_none is not None:
            c = case_or_none
            N, K, weight_bits, quant_op, group_size = c.N, c.K, c.bits, c.quant_op, c.group_size
            weights, scale, zeros, bias = c.w, c.scale, c.zero, c.bias
            max_M = max(max_M, c.M)
        self.N, self.K, self.max_M = int(N), int(K), int(max_M)
        w = np.ascontiguousarray(weights)
        s = np.ascontiguousarray(scale, dtype=np.float16)
        z = None if zeros is None else np.ascontiguousarray(zeros, dtype=np.float16)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
        h = C.c_void_p()
        p = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
        check(_lib.load().mgv_linear_create(C.byref(h), self.N, self.K, int(weight_bits), int(quant_op),
                                            int(group_size), int(layout), p(w), p(s), p(z), p(b),
                                            self.max_M))
        self._h = h

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, M: int = 1,
                     variant: Variant = Variant.AUTO) -> None:
        """x_host fp16 [M, K] and out_host fp16 [M, N] are HOST tensors (pinned or pageable)."""
        check(_lib.load().mgv_linear_forward_host(self._h, x_host.data_ptr(), out_host.data_ptr(),
                                                  int(M), int(variant)))

    def forward(self, x: torch.Tensor, out: torch.Tensor, M: int = 1,
                variant: Variant = Variant.AUTO, stream=None) -> None:
        check(_lib.load().mgv_linear_forward(self._h, _dev_ptr(x, "x"), _dev_ptr(out, "out"), int(M),
                                             int(variant), _stream_ptr(stream)))

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.load().mgv_linear_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
