"""mixed_gemv_b200: weight-only-quantised (int4/int8 x fp16) GEMV for B200 (sm_100a).

The product is ``libmixed_gemv_b200.so`` (hand-written CUDA behind the C ABI declared in
``include/mixed_gemv_b200.h``).  This package is the thin host side: a ctypes binding that
mirrors the reference's interface (``api``), seeded synthetic inputs (``synth``) and the
multi-GPU sharding helpers (``sharded``).  There is no CPU or PyTorch fallback.
"""
from .enums import LayoutType, QuantType, Status, Variant, WeightOnlyQuantOp, has_zero, is_finegrained
from ._lib import MgvError

__all__ = ["LayoutType", "QuantType", "Status", "Variant", "WeightOnlyQuantOp", "has_zero",
           "is_finegrained", "MgvError"]
