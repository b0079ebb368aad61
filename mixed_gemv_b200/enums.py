"""Selector enums; numeric values equal the reference's so they can cross the C ABI as ints."""
from enum import IntEnum


class WeightOnlyQuantOp(IntEnum):
    """gemv/weight_only_quant_op.h:12-18"""
    UNDEFINED = 0
    PER_COLUMN_SCALE_ONLY = 1
    FINEGRAINED_SCALE_ONLY = 2
    FINEGRAINED_SCALE_AND_ZEROS = 3


def is_finegrained(op) -> bool:
    """gemv/weight_only_quant_op.h:21-24"""
    return WeightOnlyQuantOp(op) in (WeightOnlyQuantOp.FINEGRAINED_SCALE_ONLY,
                                     WeightOnlyQuantOp.FINEGRAINED_SCALE_AND_ZEROS)


def has_zero(op) -> bool:
    """gemv/weight_only_quant_op.h:27-30"""
    return WeightOnlyQuantOp(op) == WeightOnlyQuantOp.FINEGRAINED_SCALE_AND_ZEROS


class QuantType(IntEnum):
    """utils/type_base.h:7-11"""
    W8_A16 = 0
    W4_A16 = 1
    W4_AFP8 = 2


class LayoutType(IntEnum):
    """utils/type_base.h:13-16"""
    kRowMajor = 0
    kColumnMajor = 1


class Status(IntEnum):
    """mgv_status of include/mixed_gemv_b200.h"""
    OK = 0
    INVALID_ARGUMENT = 1
    UNSUPPORTED = 2
    MISALIGNED = 3
    WORKSPACE_TOO_SMALL = 4
    CUDA_ERROR = 5
    DEVICE_TIMEOUT = 6


class Variant(IntEnum):
    """Kernel family selector of mgv_gemv_args.variant."""
    AUTO = 0
    SIMT = 1
    MMA = 2
