"""Runs the reference-style C++ driver (tests/cpp/adaptor_driver.cpp over include/mixed_gemv_b200.hpp)
on the GPU and checks its output against the CPU checker: preprocess weights, preprocess
zero-points, device_gemv() -- the sequence of the reference's mixed_gemv_test.cu."""
import subprocess

import numpy as np
import pytest

from mixed_gemv_b200 import synth
from mixed_gemv_b200.enums import WeightOnlyQuantOp as Q
from tests import cpp_util
from tests.gpu_util import oracle_out

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    return cpp_util.build_driver(str(tmp_path_factory.mktemp("cpp")))


@pytest.mark.parametrize("bits,op,group,batch,bias", [(4, Q.FINEGRAINED_SCALE_AND_ZEROS, 128, 1, False),
                                                       (4, Q.FINEGRAINED_SCALE_ONLY, 64, 3, True),
                                                       (8, Q.PER_COLUMN_SCALE_ONLY, 0, 2, True)])
def test_driver_matches_the_checker(cuda_lib, driver, tmp_path, bits, op, group, batch, bias):
    K, N = 1024, 512
    c = synth.make_case(batch, N, K, bits=bits, quant_op=op, group_size=group or K, zeros="int8" if op == Q.FINEGRAINED_SCALE_AND_ZEROS else "none",
                        bias=bias, seed=21)
    inp, outp = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([N, batch, K, bits, int(op), group or K, int(bias), 0], dtype=np.int32).tobytes())
        f.write(np.ascontiguousarray(c.w).tobytes())
        f.write(np.ascontiguousarray(c.x).tobytes())
        f.write(np.ascontiguousarray(c.scale).tobytes())
        if op == Q.FINEGRAINED_SCALE_AND_ZEROS:
            f.write(np.ascontiguousarray(c.zero_i8).tobytes())
        if bias:
            f.write(np.ascontiguousarray(c.bias).tobytes())
    r = subprocess.run([driver, str(inp), str(outp)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "ok" in r.stdout                       # and the refused call was reported, not fatal
    assert "invalid argument" in r.stderr or "unsupported" in r.stderr
    got = np.fromfile(outp, dtype=np.float16).reshape(batch, N)
    ok, max_abs, max_rel = synth.check_close(got, oracle_out(c), c)
    assert ok, (max_abs, max_rel)
