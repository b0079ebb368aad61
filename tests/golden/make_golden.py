"""Generates tests/golden/*.npz by running the REFERENCE'S OWN host code (oracle/_ref, built
from the reference's headers by oracle/Makefile) on seeded inputs.

Run where the reference tree is mounted:  python tests/golden/make_golden.py
The fixtures are committed; the tests read them everywhere, also where the reference and the
shim are absent.  Inputs are stored next to the outputs so that a fixture does not depend on
the generator's random stream.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def pack(u):
    u8 = np.ascontiguousarray(u, dtype=np.int8).ravel().view(np.uint8)
    return ((u8[0::2] & 0xF) | ((u8[1::2] & 0xF) << 4)).astype(np.uint8)


def preprocess_cases():
    out = {}
    specs = [  # name, shape, layout, quant_type
        ("w4_col_128x64", (128, 64), oracle.COLUMN_MAJOR, oracle.W4_A16),
        ("w4_row_128x64", (128, 64), oracle.ROW_MAJOR, oracle.W4_A16),
        ("w4_col_64x20", (64, 20), oracle.COLUMN_MAJOR, oracle.W4_A16),
        ("w4_col_3d_2x64x64", (2, 64, 64), oracle.COLUMN_MAJOR, oracle.W4_A16),
        ("w4_row_3d_2x64x64", (2, 64, 64), oracle.ROW_MAJOR, oracle.W4_A16),
        ("w8_col_64x32", (64, 32), oracle.COLUMN_MAJOR, oracle.W8_A16),
        ("w8_row_64x32", (64, 32), oracle.ROW_MAJOR, oracle.W8_A16),
        ("w8_col_72x6", (72, 6), oracle.COLUMN_MAJOR, oracle.W8_A16),
    ]
    for i, (name, shape, layout, qt) in enumerate(specs):
        g = rng(100 + i)
        n = int(np.prod(shape))
        if qt == oracle.W4_A16:
            src = pack(g.integers(-8, 8, size=n, dtype=np.int8))
        else:
            src = g.integers(-128, 128, size=n, dtype=np.int8).view(np.uint8)
        dst = oracle.ref_preprocess_weights(src, shape, layout, qt)
        out[name + "__src"] = src
        out[name + "__dst"] = dst
        out[name + "__meta"] = np.array(list(shape) + [layout, qt], dtype=np.int64)
    return out


def misc_cases():
    g = rng(7)
    scales = g.uniform(0.001, 0.3, size=256).astype(np.float16)
    zeros = g.integers(-8, 8, size=256, dtype=np.int8)
    unpacked = g.integers(-8, 8, size=512, dtype=np.int8)
    packed = oracle.ref_pack_int4(unpacked)
    return {
        "zeros__scales": scales, "zeros__zeros": zeros,
        "zeros__out": oracle.ref_preprocess_zeros(scales, zeros),
        "pack__unpacked": unpacked, "pack__packed": packed,
        "pack__roundtrip": oracle.ref_unpack_int4(packed),
    }


def gemv_cases():
    out = {}
    specs = [  # name, N, K, group, zeros, bias, scale range
        ("percol", 64, 256, 256, False, False, (0.001, 0.01)),
        ("g128", 64, 256, 128, False, False, (0.001, 0.02)),
        ("g64_zeros_bias", 48, 256, 64, True, True, (0.1, 0.3)),
        ("g128_zeros_wide", 36, 1024, 128, True, False, (0.001, 0.02)),
    ]
    for i, (name, N, K, group, zeros, bias, sr) in enumerate(specs):
        g = rng(200 + i)
        w = g.integers(-8, 8, size=(N, K), dtype=np.int8)
        x = g.uniform(-1, 1, size=K).astype(np.float16)
        scale = g.uniform(sr[0], sr[1], size=(K // group, N)).astype(np.float16)
        z = g.integers(-8, 8, size=(K // group, N), dtype=np.int8) if zeros else None
        b = g.uniform(-0.1, 0.1, size=N).astype(np.float16) if bias else None
        y = oracle.ref_host_gemv_int4(pack(w), x, scale, z, b, group_size=group)
        out[name + "__w"] = w
        out[name + "__x"] = x
        out[name + "__scale"] = scale
        if z is not None:
            out[name + "__zero_i8"] = z
        if b is not None:
            out[name + "__bias"] = b
        out[name + "__out"] = y
        out[name + "__meta"] = np.array([N, K, group], dtype=np.int64)
    return out


if __name__ == "__main__":
    oracle.build(ref=True)
    if not oracle.have_ref():
        sys.exit("the reference shim could not be built here (reference tree or CUTLASS headers absent)")
    np.savez_compressed(os.path.join(HERE, "preprocess.npz"), **preprocess_cases())
    np.savez_compressed(os.path.join(HERE, "misc.npz"), **misc_cases())
    np.savez_compressed(os.path.join(HERE, "gemv_int4.npz"), **gemv_cases())
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
