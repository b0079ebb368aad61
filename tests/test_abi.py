"""CPU tests of the drop-in boundary: the library loads without a GPU and exports exactly the
symbols the header declares; the enums carry the reference's numeric values."""
import ctypes
import os
import re

import pytest

from mixed_gemv_b200 import _lib, enums

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mixed_gemv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mgv_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    assert _declared_symbols() == sorted(_lib.EXPORTS)


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.load()
    for name in _declared_symbols():
        assert hasattr(lib, name), name
    assert lib.mgv_version() >= 100
    assert lib.mgv_status_string(0) == b"ok"
    assert lib.mgv_status_string(6) == b"device-side wait timed out"


def test_args_struct_matches_the_header_layout():
    lib = _lib.load()
    a = _lib.GemvArgs()
    lib.mgv_gemv_args_init(ctypes.byref(a))
    assert a.struct_size == ctypes.sizeof(_lib.GemvArgs)
    assert a.alpha == 1.0 and a.beta == 1.0 and a.batch_count == 1 and a.variant == 0


def test_enum_values_equal_the_reference():
    # gemv/weight_only_quant_op.h:12-18, utils/type_base.h:7-16
    assert [int(v) for v in enums.WeightOnlyQuantOp] == [0, 1, 2, 3]
    assert (enums.QuantType.W8_A16, enums.QuantType.W4_A16, enums.QuantType.W4_AFP8) == (0, 1, 2)
    assert (enums.LayoutType.kRowMajor, enums.LayoutType.kColumnMajor) == (0, 1)
    assert enums.is_finegrained(2) and enums.is_finegrained(3) and not enums.is_finegrained(1)
    assert enums.has_zero(3) and not enums.has_zero(2)
    text = open(os.path.join(ROOT, "include", "mixed_gemv_b200.h")).read()
    for name, val in [("MGV_QUANT_PER_COLUMN_SCALE_ONLY", 1), ("MGV_QUANT_FINEGRAINED_SCALE_ONLY", 2),
                      ("MGV_QUANT_FINEGRAINED_SCALE_AND_ZEROS", 3), ("MGV_W8_A16", 0), ("MGV_W4_A16", 1),
                      ("MGV_LAYOUT_ROW_MAJOR", 0), ("MGV_LAYOUT_COLUMN_MAJOR", 1)]:
        assert re.search(rf"\b{name} = {val}\b", text), name


def test_argument_errors_need_no_gpu():
    """Checks made before any CUDA call return a status and a message instead of exiting."""
    lib = _lib.load()
    shape = (ctypes.c_size_t * 2)(64, 64)
    assert lib.mgv_preprocess_weights(None, None, shape, 2, 1, 2, None) == enums.Status.UNSUPPORTED
    assert b"W4_AFP8" in lib.mgv_last_error()
    assert lib.mgv_preprocess_weights(None, None, shape, 4, 1, 1, None) == enums.Status.INVALID_ARGUMENT
    shape = (ctypes.c_size_t * 2)(64, 6)
    assert lib.mgv_preprocess_weights(None, None, shape, 2, 1, 1, None) == enums.Status.INVALID_ARGUMENT
    assert lib.mgv_pack_int4(None, None, 3, None) == enums.Status.INVALID_ARGUMENT


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "mixed_gemv_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.lower(), (base, f)
