"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

The reference draws its test inputs from an unseeded ``std::random_device``
(utils/initializer.h:37-38), so nothing it produces is reproducible; these generators use
numpy's Philox with an explicit seed instead.  Distributions follow the reference test
(mixed_gemv_test.cu:200-234: weights uniform over the signed range, activations uniform in
[-1, 1], scales uniform, int8 zero-points uniform over [-8, 7]) and the benchmark configs.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .enums import WeightOnlyQuantOp


@dataclass
class Case:
    """One GEMV problem on the host.  ``w`` is NOT preprocessed: element (n, k) is at
    linear index n*K + k (LayoutType.kColumnMajor of a {K, N} matrix), packed two per byte
    for 4-bit weights."""
    M: int
    N: int
    K: int
    bits: int
    quant_op: WeightOnlyQuantOp
    group_size: int
    w: np.ndarray                 # uint8 [N*K/2] (4 bit) or int8 [N, K] (8 bit)
    w_unpacked: np.ndarray        # int8 [N, K]
    x: np.ndarray                 # fp16 [M, K]
    scale: np.ndarray             # fp16 [G, N]
    zero: np.ndarray | None       # fp16 [G, N] additive (device format) or None
    zero_i8: np.ndarray | None    # int8 [G, N] zero-points the additive zeros came from, or None
    bias: np.ndarray | None       # fp16 [N] or None
    name: str = ""
    extra: dict = field(default_factory=dict)

    @property
    def groups(self) -> int:
        return self.K // self.group_size

    def algorithmic_bytes(self) -> int:
        """Bytes one call must move, each operand counted once."""
        g = self.groups
        b = self.K * self.N * self.bits // 8 + g * self.N * 2
        if self.zero is not None:
            b += g * self.N * 2
        b += self.M * self.K * 2 + self.M * self.N * 2
        if self.bias is not None:
            b += self.N * 2
        return b


def pack_int4_np(unpacked: np.ndarray) -> np.ndarray:
    """Two int4 per byte, even index in the low nibble (utils/preprocess.h:79-80)."""
    u = np.ascontiguousarray(unpacked, dtype=np.int8).ravel().view(np.uint8)
    return ((u[0::2] & 0xF) | ((u[1::2] & 0xF) << 4)).astype(np.uint8)


def make_case(M, N, K, *, bits=4, quant_op=WeightOnlyQuantOp.FINEGRAINED_SCALE_ONLY,
              group_size=128, x_dist="uniform", scale_range=(0.001, 0.02), zeros="none",
              zero_range=(-0.05, 0.05), bias=False, bias_range=(-0.1, 0.1), seed=0,
              name="") -> Case:
    """``zeros``: "none", "f16" (fp16 additive zeros drawn directly) or "int8" (int8
    zero-points in [-8, 7], converted as utils/preprocess.h:94-101 does)."""
    quant_op = WeightOnlyQuantOp(quant_op)
    if quant_op == WeightOnlyQuantOp.PER_COLUMN_SCALE_ONLY:
        group_size = K
    rng = np.random.Generator(np.random.Philox(seed))
    lo, hi = (-8, 7) if bits == 4 else (-128, 127)
    w_unpacked = rng.integers(lo, hi + 1, size=(N, K), dtype=np.int8)
    w = pack_int4_np(w_unpacked) if bits == 4 else w_unpacked.copy()
    if x_dist == "uniform":
        x = rng.uniform(-1.0, 1.0, size=(M, K)).astype(np.float16)
    else:
        x = rng.standard_normal(size=(M, K)).astype(np.float16)
    G = K // group_size
    scale = rng.uniform(scale_range[0], scale_range[1], size=(G, N)).astype(np.float16)
    zero = zero_i8 = None
    if quant_op == WeightOnlyQuantOp.FINEGRAINED_SCALE_AND_ZEROS:
        if zeros == "int8":
            zero_i8 = rng.integers(-8, 8, size=(G, N), dtype=np.int8)
            zero = ((-zero_i8.astype(np.float32)).astype(np.float16).astype(np.float32)
                    * scale.astype(np.float32)).astype(np.float16)
        else:
            zero = rng.uniform(zero_range[0], zero_range[1], size=(G, N)).astype(np.float16)
    b = rng.uniform(bias_range[0], bias_range[1], size=(N,)).astype(np.float16) if bias else None
    return Case(M=M, N=N, K=K, bits=bits, quant_op=quant_op, group_size=group_size, w=w,
                w_unpacked=w_unpacked, x=x, scale=scale, zero=zero, zero_i8=zero_i8, bias=b,
                name=name)


# The benchmark configs (names are used by bench.py and the parity tests).
def config(name: str, M: int = 1, seed: int = 0, N: int | None = None, K: int | None = None) -> Case:
    Q = WeightOnlyQuantOp
    if name == "c1_int8_percol_bias":
        return make_case(M, N or 4096, K or 4096, bits=8, quant_op=Q.PER_COLUMN_SCALE_ONLY,
                         scale_range=(0.001, 0.01), bias=True, seed=seed, name=name)
    if name == "c2_int4_g128":
        return make_case(M, N or 11008, K or 4096, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY,
                         group_size=128, seed=seed, name=name)
    if name == "c3_int4_g64_zeros_bias":
        return make_case(M, N or 28672, K or 8192, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS,
                         group_size=64, x_dist="normal", zeros="f16", bias=True, seed=seed,
                         name=name)
    llama = {"c4_qkv": (4096, 12288), "c4_oproj": (4096, 4096), "c4_gateup": (4096, 22016),
             "c4_down": (11008, 4096), "c5_gateup": (8192, 57344), "c5_down": (28672, 8192)}
    if name in llama:
        k, n = llama[name]
        return make_case(M, N or n, K or k, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY,
                         group_size=128, x_dist="normal", seed=seed, name=name)
    if name == "ref_shape":
        # the shape, mode and group size of the reference's own test driver (mixed_gemv_test.cu:84,187,191),
        # with int8 zero-points converted as its ZeroPointPreprocessor does (:231-239)
        return make_case(M, N or 151936, K or 2048, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS,
                         group_size=128, x_dist="uniform", scale_range=(0.1, 0.3), zeros="int8", seed=seed, name=name)
    raise KeyError(name)


CONFIG_NAMES = ["c1_int8_percol_bias", "c2_int4_g128", "c3_int4_g64_zeros_bias", "c4_qkv",
                "c4_oproj", "c4_gateup", "c4_down", "c5_gateup", "c5_down"]


def tolerance(case: Case):
    """(rtol, atol): max relative error 1e-2, max absolute error 1e-2*sqrt(K)*max|scale|."""
    return 1e-2, 1e-2 * float(np.sqrt(case.K)) * float(np.abs(case.scale.astype(np.float32)).max())


def check_close(got: np.ndarray, want: np.ndarray, case: Case):
    """The two stated bounds combined the way numpy.allclose combines them: every element must
    satisfy |got - want| <= atol + rtol*|want|.  (Alone, the absolute bound can be finer than
    one fp16 ulp of a large output, and the relative bound is meaningless for outputs that
    cancel to nearly zero.)  Returns (ok, max_abs, max_rel); max_rel is taken over the elements
    whose reference magnitude is at least atol."""
    rtol, atol = tolerance(case)
    g = np.asarray(got, dtype=np.float32)
    w = np.asarray(want, dtype=np.float32)
    err = np.abs(g - w)
    max_abs = float(err.max()) if err.size else 0.0
    big = np.abs(w) >= atol
    max_rel = float((err[big] / np.abs(w[big])).max()) if big.any() else 0.0
    ok = bool(np.isfinite(g).all() and (err <= atol + rtol * np.abs(w)).all())
    return ok, max_abs, max_rel
