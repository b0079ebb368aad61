"""GPU parity: the preprocessing kernels against the CPU checker and the reference's golden
vectors, bit for bit, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import oracle
from mixed_gemv_b200 import api, synth
from mixed_gemv_b200.enums import LayoutType, QuantType, Status
from mixed_gemv_b200._lib import MgvError

pytestmark = pytest.mark.gpu


def _gpu_preprocess(src: np.ndarray, shape, layout, qt) -> np.ndarray:
    s = torch.from_numpy(np.ascontiguousarray(src).view(np.uint8).ravel().copy()).cuda()
    d = torch.full_like(s, 0xA5)
    api.MixedGemvWeightPreprocessor.run(d, s, shape, LayoutType(layout), QuantType(qt), False)
    torch.cuda.synchronize()
    return d.cpu().numpy()


def test_golden_vectors(cuda_lib, golden):
    g = golden["preprocess"]
    names = sorted(k[:-5] for k in g.files if k.endswith("__dst"))
    for name in names:
        meta = g[name + "__meta"]
        shape, layout, qt = [int(v) for v in meta[:-2]], int(meta[-2]), int(meta[-1])
        got = _gpu_preprocess(g[name + "__src"], shape, layout, qt)
        assert np.array_equal(got, g[name + "__dst"]), name


@pytest.mark.parametrize("bits,K,N", [(4, 8, 4), (4, 64, 64), (4, 72, 20), (4, 4096, 1024), (4, 2048, 4100),
                                      (8, 8, 2), (8, 64, 64), (8, 200, 66), (8, 1024, 2048)])
def test_column_major_random(cuda_lib, bits, K, N):
    rng = np.random.Generator(np.random.Philox(K * 7 + N))
    qt = oracle.W4_A16 if bits == 4 else oracle.W8_A16
    src = rng.integers(0, 256, size=K * N * bits // 8, dtype=np.uint8)
    want = oracle.preprocess_weights(src, (K, N), oracle.COLUMN_MAJOR, qt)
    assert np.array_equal(_gpu_preprocess(src, (K, N), oracle.COLUMN_MAJOR, qt), want)


@pytest.mark.parametrize("bits,K,N", [(4, 64, 64), (4, 192, 320), (4, 4096, 1024), (8, 32, 32), (8, 96, 160),
                                      (8, 1024, 2048)])
def test_row_major_random_and_layout_equivalence(cuda_lib, bits, K, N):
    rng = np.random.Generator(np.random.Philox(K * 11 + N))
    qt = oracle.W4_A16 if bits == 4 else oracle.W8_A16
    lo, hi = (-8, 8) if bits == 4 else (-128, 128)
    w = rng.integers(lo, hi, size=(N, K), dtype=np.int8)
    to_bytes = (lambda a: synth.pack_int4_np(a)) if bits == 4 else (lambda a: np.ascontiguousarray(a).view(np.uint8).ravel())
    col, row = to_bytes(w), to_bytes(np.ascontiguousarray(w.T))
    want = oracle.preprocess_weights(row, (K, N), oracle.ROW_MAJOR, qt)
    got_row = _gpu_preprocess(row, (K, N), oracle.ROW_MAJOR, qt)
    got_col = _gpu_preprocess(col, (K, N), oracle.COLUMN_MAJOR, qt)
    assert np.array_equal(got_row, want)
    assert np.array_equal(got_col, want)      # both input layouts give byte-identical output


def test_three_dimensional_experts(cuda_lib):
    rng = np.random.Generator(np.random.Philox(21))
    for bits, qt in ((4, oracle.W4_A16), (8, oracle.W8_A16)):
        E, K, N = 3, 128, 192
        src = rng.integers(0, 256, size=E * K * N * bits // 8, dtype=np.uint8)
        for layout in (oracle.COLUMN_MAJOR, oracle.ROW_MAJOR):
            want = oracle.preprocess_weights(src, (E, K, N), layout, qt)
            assert np.array_equal(_gpu_preprocess(src, (E, K, N), layout, qt), want)


def test_n_shards_are_contiguous_byte_ranges(cuda_lib):
    """preprocess(W)[rows n0:n1] == preprocess(W[n0:n1]) for n0, n1 multiples of the interleave."""
    rng = np.random.Generator(np.random.Philox(22))
    K, N = 256, 512
    w = rng.integers(-8, 8, size=(N, K), dtype=np.int8)
    full = _gpu_preprocess(synth.pack_int4_np(w), (K, N), oracle.COLUMN_MAJOR, oracle.W4_A16)
    for n0, n1 in ((0, 128), (128, 384), (384, 512)):
        part = _gpu_preprocess(synth.pack_int4_np(w[n0:n1]), (K, n1 - n0), oracle.COLUMN_MAJOR, oracle.W4_A16)
        assert np.array_equal(part, full[n0 * K // 2:n1 * K // 2])


def test_pack_unpack_and_zero_points(cuda_lib, golden):
    g = golden["misc"]
    u = torch.from_numpy(g["pack__unpacked"].copy()).cuda()
    p = torch.zeros(u.numel() // 2, dtype=torch.uint8, device="cuda")
    api.SubBytePacker.pack(p, u, u.numel())
    assert np.array_equal(p.cpu().numpy(), g["pack__packed"])
    back = torch.zeros_like(u)
    api.SubBytePacker.unpack(back, p, p.numel())
    assert np.array_equal(back.cpu().numpy(), g["pack__unpacked"])       # mixed_gemv_test.cu:211-217
    s = torch.from_numpy(g["zeros__scales"].copy()).cuda()
    z = torch.from_numpy(g["zeros__zeros"].copy()).cuda()
    out = torch.zeros_like(s)
    api.ZeroPointPreprocessor.neg_zero_point_multiplies_scale(out, s, z, s.numel())
    assert np.array_equal(out.cpu().numpy().view(np.uint16), g["zeros__out"].view(np.uint16))
    # a larger random case against the CPU checker
    rng = np.random.Generator(np.random.Philox(23))
    sc = rng.uniform(1e-4, 0.5, size=100003).astype(np.float16)
    zp = rng.integers(-128, 128, size=100003, dtype=np.int8)
    out = torch.zeros(sc.size, dtype=torch.float16, device="cuda")
    api.ZeroPointPreprocessor.neg_zero_point_multiplies_scale(out, torch.from_numpy(sc).cuda(), torch.from_numpy(zp).cuda(), sc.size)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), oracle.preprocess_zeros(sc, zp).view(np.uint16))


def test_empty_and_refused_inputs(cuda_lib):
    d = torch.zeros(16, dtype=torch.uint8, device="cuda")
    s = torch.zeros(16, dtype=torch.uint8, device="cuda")
    api.MixedGemvWeightPreprocessor.run(d, s, (0, 64), LayoutType.kColumnMajor, QuantType.W4_A16)   # empty: no-op
    api.SubBytePacker.pack(d, s, 0)
    for shape, layout, qt, status in [((64, 6), 1, 1, Status.INVALID_ARGUMENT), ((60, 8), 1, 1, Status.INVALID_ARGUMENT),
                                      ((64, 32), 0, 1, Status.INVALID_ARGUMENT), ((64, 64), 1, 2, Status.UNSUPPORTED),
                                      ((64, 3), 1, 0, Status.INVALID_ARGUMENT)]:
        with pytest.raises(MgvError) as e:
            api.MixedGemvWeightPreprocessor.run(d, s, shape, LayoutType(layout), QuantType(qt))
        assert e.value.status == status
    with pytest.raises(MgvError):
        api.MixedGemvWeightPreprocessor.run(d, torch.zeros(16, dtype=torch.uint8), (8, 4), LayoutType.kColumnMajor, QuantType.W4_A16)
