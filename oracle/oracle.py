"""ctypes front-end to the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this module; the shipped package never does and has no CPU fallback.

Three libraries sit behind it:

* ``_build/libmgv_oracle.so`` -- the plain-C restatement (``mgv_oracle.c``), always available
  after ``make -C oracle oracle``.
* ``_ref/libmgv_ref.so`` -- the reference's own host code compiled from its headers
  (``ref_shim.cpp``); present only where it was built.  ``have_ref()`` tells.
* ``_ref/libmgv_ref_cuda.so`` -- the reference's own CUDA kernel recompiled for sm_100a
  (``ref_shim_cuda.cu``): a second checker for the device path and the "reference kernel on this
  GPU" figure of ``bench.py``.  ``have_ref_cuda()`` tells.

fp16 arrays are numpy ``float16``; packed int4 weights are ``uint8`` with element ``i`` in
byte ``i//2``, even ``i`` in the low nibble (utils/preprocess.h:79-80).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "_build", "libmgv_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libmgv_ref.so")
_REF_CUDA_SO = os.path.join(_HERE, "_ref", "libmgv_ref_cuda.so")

ZERO_NONE, ZERO_INT8, ZERO_F16 = 0, 1, 2
W8_A16, W4_A16, W4_AFP8 = 0, 1, 2
ROW_MAJOR, COLUMN_MAJOR = 0, 1

_lib = None
_ref = None
_ref_cuda = None


def build(ref: bool = True) -> None:
    """Compile the checkers (the reference shim only where its sources exist)."""
    targets = ["oracle"] + (["ref", "ref_cuda"] if ref else [])
    subprocess.run(["make", "-s", "-C", _HERE] + targets, check=True)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            build(ref=False)
        _lib = C.CDLL(_ORACLE_SO)
        _lib.mgv_oracle_h2f.restype = C.c_float
        _lib.mgv_oracle_h2f.argtypes = [C.c_uint16]
        _lib.mgv_oracle_f2h.restype = C.c_uint16
        _lib.mgv_oracle_f2h.argtypes = [C.c_float]
        _lib.mgv_oracle_preprocess_weights.argtypes = [
            C.c_void_p, C.c_void_p, C.POINTER(C.c_size_t), C.c_int, C.c_int, C.c_int]
        _lib.mgv_oracle_preprocess_zeros.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        _lib.mgv_oracle_pack_int4.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        _lib.mgv_oracle_unpack_int4.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        _lib.mgv_oracle_gemv.argtypes = [
            C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int64,
            C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_float, C.c_void_p,
            C.c_int64, C.c_void_p, C.c_int]
        _lib.mgv_oracle_read_preprocessed.argtypes = [C.c_void_p] + [C.c_int] * 5
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_SO)


def ref():
    global _ref
    if _ref is None:
        if not have_ref():
            raise RuntimeError("oracle/_ref/libmgv_ref.so is not built on this machine")
        _ref = C.CDLL(_REF_SO)
        _ref.ref_preprocess_weights.argtypes = [
            C.c_void_p, C.c_void_p, C.POINTER(C.c_size_t), C.c_int, C.c_int, C.c_int]
        _ref.ref_preprocess_zeros.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        _ref.ref_pack_int4.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        _ref.ref_unpack_int4.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        _ref.ref_host_gemv_int4.argtypes = [C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 6 + [C.c_int]
    return _ref


def max_threads() -> int:
    return int(lib().mgv_oracle_max_threads())


# ---------------------------------------------------------------- C restatement ----------

def pack_int4(unpacked: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(unpacked, dtype=np.int8).ravel()
    out = np.empty(u.size // 2, dtype=np.uint8)
    lib().mgv_oracle_pack_int4(_ptr(out), _ptr(u), u.size)
    return out


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    p = np.ascontiguousarray(packed, dtype=np.uint8).ravel()
    out = np.empty(p.size * 2, dtype=np.int8)
    lib().mgv_oracle_unpack_int4(_ptr(out), _ptr(p), p.size)
    return out


def _shape_arg(shape):
    arr = (C.c_size_t * len(shape))(*[int(s) for s in shape])
    return arr, len(shape)


def preprocess_weights(src: np.ndarray, shape, layout: int, quant_type: int) -> np.ndarray:
    s = np.ascontiguousarray(src, dtype=np.uint8).ravel()
    out = np.empty_like(s)
    arr, rank = _shape_arg(shape)
    rc = lib().mgv_oracle_preprocess_weights(_ptr(out), _ptr(s), arr, rank, layout, quant_type)
    if rc:
        raise ValueError(f"oracle preprocess_weights refused the input (code {rc})")
    return out


def preprocess_zeros(scales: np.ndarray, zeros: np.ndarray) -> np.ndarray:
    s = np.ascontiguousarray(scales, dtype=np.float16).ravel()
    z = np.ascontiguousarray(zeros, dtype=np.int8).ravel()
    out = np.empty_like(s)
    lib().mgv_oracle_preprocess_zeros(_ptr(out), _ptr(s), _ptr(z), s.size)
    return out.reshape(np.shape(scales))


def gemv(w, x, scale, *, bits, group_size, zero=None, bias=None, alpha=1.0, beta=1.0,
         n_threads=1, want_f32=False):
    """host/mixed_gemv.h:82-104 generalised.  ``w``: un-preprocessed [N,K] weights
    (packed uint8 for 4 bits, int8 for 8 bits); ``x``: [M,K] fp16; ``scale``: [G,N] fp16;
    ``zero``: None, int8 [G,N] zero-points or fp16 [G,N] additive zeros; ``bias``: [N]."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    if x.ndim == 1:
        x = x[None, :]
    M, K = x.shape
    scale = np.ascontiguousarray(scale, dtype=np.float16)
    N = scale.shape[-1]
    wb = np.ascontiguousarray(w).view(np.uint8).ravel()
    assert wb.size == N * K * bits // 8, (wb.size, N, K, bits)
    if zero is None:
        zk, zz = ZERO_NONE, None
    elif zero.dtype == np.int8:
        zk, zz = ZERO_INT8, np.ascontiguousarray(zero)
    else:
        zk, zz = ZERO_F16, np.ascontiguousarray(zero, dtype=np.float16)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    out = np.empty((M, N), dtype=np.float16)
    acc = np.empty((M, N), dtype=np.float32) if want_f32 else None
    rc = lib().mgv_oracle_gemv(M, N, K, bits, group_size, _ptr(wb), _ptr(x), K, _ptr(scale),
                               _ptr(zz), zk, _ptr(b), alpha, beta, _ptr(out), N, _ptr(acc),
                               n_threads)
    if rc:
        raise ValueError(f"oracle gemv refused the input (code {rc})")
    return (out, acc) if want_f32 else out


def read_preprocessed(pre: np.ndarray, N: int, K: int, bits: int, n: int, k: int) -> int:
    p = np.ascontiguousarray(pre, dtype=np.uint8).ravel()
    return int(lib().mgv_oracle_read_preprocessed(_ptr(p), N, K, bits, n, k))


# ---------------------------------------------------------------- reference shim ---------

def ref_pack_int4(unpacked):
    u = np.ascontiguousarray(unpacked, dtype=np.int8).ravel()
    out = np.zeros(u.size // 2, dtype=np.uint8)
    ref().ref_pack_int4(_ptr(out), _ptr(u), u.size)
    return out


def ref_unpack_int4(packed):
    p = np.ascontiguousarray(packed, dtype=np.uint8).ravel()
    out = np.empty(p.size * 2, dtype=np.int8)
    ref().ref_unpack_int4(_ptr(out), _ptr(p), p.size)
    return out


def ref_preprocess_weights(src, shape, layout, quant_type):
    s = np.ascontiguousarray(src, dtype=np.uint8).ravel()
    out = np.empty_like(s)
    arr, rank = _shape_arg(shape)
    rc = ref().ref_preprocess_weights(_ptr(out), _ptr(s), arr, rank, layout, quant_type)
    if rc:
        raise ValueError(f"reference preprocess would exit (code {rc})")
    return out


def ref_preprocess_zeros(scales, zeros):
    s = np.ascontiguousarray(scales, dtype=np.float16).ravel()
    z = np.ascontiguousarray(zeros, dtype=np.int8).ravel()
    out = np.empty_like(s)
    ref().ref_preprocess_zeros(_ptr(out), _ptr(s), _ptr(z), s.size)
    return out.reshape(np.shape(scales))


def ref_host_gemv_int4(w_packed, x, scale, zero_i8=None, bias=None, *, group_size, n_threads=1):
    """The reference's host::reference::MixedGemv (int4 weights, int8 zero-points, M=1)."""
    x = np.ascontiguousarray(x, dtype=np.float16).ravel()
    K = x.size
    scale = np.ascontiguousarray(scale, dtype=np.float16)
    N = scale.shape[-1]
    wb = np.ascontiguousarray(w_packed, dtype=np.uint8).ravel()
    z = np.zeros(scale.shape, dtype=np.int8) if zero_i8 is None else np.ascontiguousarray(zero_i8, dtype=np.int8)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    out = np.empty(N, dtype=np.float16)
    rc = ref().ref_host_gemv_int4(N, K, group_size, _ptr(wb), _ptr(x), _ptr(scale), _ptr(z),
                                  _ptr(b), _ptr(out), n_threads)
    if rc:
        raise ValueError(f"reference host gemv refused the input (code {rc})")
    return out


# ------------------------------------------------- the reference's own CUDA kernel ----------

def have_ref_cuda() -> bool:
    return os.path.exists(_REF_CUDA_SO)


def ref_device_gemv(quant_op: int, weights_ptr: int, x_ptr: int, scale_ptr: int, zero_ptr, out_ptr: int, N: int, K: int,
                    group_size: int, stream: int = 0) -> None:
    """Enqueues the reference's GemvAdaptor (``_ref/libmgv_ref_cuda.so``: its kernel recompiled for
    sm_100a in the configuration of its test driver) on DEVICE pointers: 4-bit preprocessed
    weights, one activation row, fp16 scales (and additive zeros for quant_op 3), no bias."""
    global _ref_cuda
    if _ref_cuda is None:
        if not have_ref_cuda():
            raise RuntimeError("oracle/_ref/libmgv_ref_cuda.so is not built on this machine")
        _ref_cuda = C.CDLL(_REF_CUDA_SO)
        _ref_cuda.ref_device_gemv.argtypes = [C.c_int] + [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p]
    rc = _ref_cuda.ref_device_gemv(int(quant_op), weights_ptr, x_ptr, scale_ptr, zero_ptr or None, out_ptr, N, K, group_size,
                                   stream or None)
    if rc:
        raise ValueError("the reference kernel cannot run this configuration (4-bit, group 64 or 128, N % 4 == 0, K % 64 == 0)")
