"""ctypes binding of libmixed_gemv_b200.so: the C ABI of include/mixed_gemv_b200.h, verbatim.

There is no fallback: if the library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

from .enums import Status

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmixed_gemv_b200.so")


class MgvError(RuntimeError):
    def __init__(self, status: int, message: str):
        self.status = Status(status) if status in Status._value2member_map_ else status
        super().__init__(f"mixed_gemv_b200: {getattr(self.status, 'name', status)}: {message}")


class GemvArgs(C.Structure):
    """mgv_gemv_args"""
    _fields_ = [
        ("struct_size", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("weight_bits", C.c_int32), ("quant_op", C.c_int32), ("group_size", C.c_int32),
        ("variant", C.c_int32), ("flags", C.c_int32), ("batch_count", C.c_int32),
        ("weights", C.c_void_p), ("x", C.c_void_p), ("scale", C.c_void_p), ("zero", C.c_void_p),
        ("bias", C.c_void_p), ("out", C.c_void_p), ("ldx", C.c_int64), ("ldd", C.c_int64),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("batch_stride_weights", C.c_int64), ("batch_stride_x", C.c_int64),
        ("batch_stride_scale", C.c_int64), ("batch_stride_bias", C.c_int64),
        ("batch_stride_out", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("n_peers", C.c_int32), ("hints", C.c_int32),
        ("peer_out", C.c_void_p * 8), ("peer_flag", C.c_void_p * 8),
        ("wait_flag", C.c_void_p), ("wait_state", C.c_void_p), ("wait_delta", C.c_uint32), ("wait_sources", C.c_uint32),
        ("prefetch", C.c_void_p), ("prefetch_bytes", C.c_size_t),
    ]


class LaunchInfo(C.Structure):
    """mgv_launch_info"""
    _fields_ = [(n, C.c_int32) for n in ("variant", "grid", "block", "stages", "smem_bytes",
                                           "tile_rows", "k_slice", "split_tiles")]


FLAG_OUT_F32_PARTIAL = 1
FLAG_ACT_RELU = 2
FLAG_ACT_SILU = 4
FLAG_PDL = 8
FLAG_GATED_SILU = 16

# mgv_gemv_args.hints
HINT_DEAL_TILES, HINT_DEAL_ITEMS, HINT_DEAL_PAIRS = 1, 2, 3
HINT_ITEM_128, HINT_ITEM_256 = 4, 8
HINT_KERNEL_GENERAL, HINT_KERNEL_STAGED, HINT_KERNEL_XREG = 16, 32, 48
HINT_ONE_LAUNCH = 64

# every symbol include/mixed_gemv_b200.h declares
EXPORTS = [
    "mgv_status_string", "mgv_last_error", "mgv_version", "mgv_pack_int4", "mgv_unpack_int4",
    "mgv_preprocess_weights", "mgv_preprocess_zeros", "mgv_gemv_args_init",
    "mgv_gemv_workspace_size", "mgv_workspace_init", "mgv_gemv", "mgv_gemv_plan_create", "mgv_gemv_plan_run",
    "mgv_gemv_plan_destroy", "mgv_gemv_static_scratch",
    "mgv_device_error_state", "mgv_window_create", "mgv_window_open", "mgv_window_close",
    "mgv_window_destroy", "mgv_wait_arrivals", "mgv_reduce_partials", "mgv_wait_reduce_partials",
    "mgv_gemv_launch_info", "mgv_linear_create", "mgv_linear_forward_host", "mgv_linear_forward",
    "mgv_linear_weights", "mgv_linear_destroy",
]

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m mixed_gemv_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    lib.mgv_status_string.restype = C.c_char_p
    lib.mgv_status_string.argtypes = [i32]
    lib.mgv_last_error.restype = C.c_char_p
    lib.mgv_version.restype = i32
    lib.mgv_pack_int4.argtypes = [vp, vp, sz, vp]
    lib.mgv_unpack_int4.argtypes = [vp, vp, sz, vp]
    lib.mgv_preprocess_weights.argtypes = [vp, vp, C.POINTER(sz), i32, i32, i32, vp]
    lib.mgv_preprocess_zeros.argtypes = [vp, vp, vp, sz, vp]
    lib.mgv_gemv_args_init.argtypes = [C.POINTER(GemvArgs)]
    lib.mgv_gemv_args_init.restype = None
    lib.mgv_gemv_workspace_size.argtypes = [C.POINTER(GemvArgs), C.POINTER(sz)]
    lib.mgv_workspace_init.argtypes = [vp, sz, vp]
    lib.mgv_gemv.argtypes = [C.POINTER(GemvArgs), vp]
    lib.mgv_gemv_static_scratch.argtypes = [C.POINTER(GemvArgs), vp]
    lib.mgv_gemv_plan_create.argtypes = [C.POINTER(GemvArgs), C.POINTER(vp)]
    lib.mgv_gemv_plan_run.argtypes = [vp, vp]
    lib.mgv_gemv_plan_destroy.argtypes = [vp]
    lib.mgv_gemv_plan_destroy.restype = None
    lib.mgv_device_error_state.argtypes = [C.POINTER(i32)]
    lib.mgv_gemv_launch_info.argtypes = [C.POINTER(GemvArgs), C.POINTER(LaunchInfo)]
    lib.mgv_linear_create.argtypes = [C.POINTER(vp), i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, i32]
    lib.mgv_linear_forward_host.argtypes = [vp, vp, vp, i32, i32]
    lib.mgv_linear_forward.argtypes = [vp, vp, vp, i32, i32, vp]
    lib.mgv_linear_weights.argtypes = [vp]
    lib.mgv_linear_weights.restype = vp
    lib.mgv_linear_destroy.argtypes = [vp]
    lib.mgv_linear_destroy.restype = None
    lib.mgv_window_create.argtypes = [C.POINTER(vp), sz, vp]
    lib.mgv_window_open.argtypes = [vp, C.POINTER(vp)]
    lib.mgv_window_close.argtypes = [vp]
    lib.mgv_window_destroy.argtypes = [vp]
    lib.mgv_wait_arrivals.argtypes = [vp, vp, C.c_uint32, C.c_uint32, vp]
    lib.mgv_reduce_partials.argtypes = [vp, sz, i32, i32, i32, C.c_longlong, vp, C.c_float, i32, vp, C.c_longlong, vp]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if name not in ("mgv_status_string", "mgv_last_error", "mgv_version", "mgv_gemv_args_init",
                        "mgv_linear_weights", "mgv_linear_destroy", "mgv_gemv_plan_destroy"):
            fn.restype = i32
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise MgvError(status, load().mgv_last_error().decode())
