"""The C++ face of the library (include/mixed_gemv_b200.hpp: the reference's class and member names
over the C ABI) compiles and links as plain C++17 against the in-tree library -- no GPU needed."""
import os

from tests import cpp_util


def test_reference_style_driver_compiles_and_links(tmp_path):
    exe = cpp_util.build_driver(str(tmp_path))
    assert os.path.exists(exe) and os.access(exe, os.X_OK)


def test_mirror_keeps_the_reference_names():
    hpp = open(os.path.join(cpp_util.ROOT, "include", "mixed_gemv_b200.hpp")).read()
    for name in ("class GemvAdaptor", "struct Arguments", "problem_size", "ref_A", "ref_B", "ref_scale", "ref_zero_point",
                 "ref_C", "ref_D", "epilogue", "group_size", "batch_count", "batch_stride_A", "batch_stride_B",
                 "batch_stride_scale", "batch_stride_C", "batch_stride_D", "initialize(", "run(", "operator()(",
                 "struct MixedGemvWeightPreprocessor", "struct ZeroPointPreprocessor", "neg_zero_point_multiplies_scale",
                 "struct SubBytePacker", "PER_COLUMN_SCALE_ONLY", "FINEGRAINED_SCALE_ONLY", "FINEGRAINED_SCALE_AND_ZEROS",
                 "kColumnMajor", "W4_A16", "W8_A16"):
        assert name in hpp, name
