"""CPU tests: the C restatement against the reference's golden vectors, against the reference's
own host code where it is built, and against closed forms of the layout."""
import numpy as np
import pytest

from oracle import oracle
from mixed_gemv_b200 import synth
from mixed_gemv_b200.enums import WeightOnlyQuantOp as Q


def _names(npz, suffix):
    return sorted(k[: -len(suffix)] for k in npz.files if k.endswith(suffix))


def test_fp16_conversions_match_numpy_exhaustively():
    lib = oracle.lib()
    # every fp16 bit pattern -> float -> back
    for h in range(0, 1 << 16, 1):
        f = np.uint16(h).view(np.float16).astype(np.float32)
        got = lib.mgv_oracle_h2f(h)
        if np.isnan(f):
            assert np.isnan(got)
            continue
        assert got == f
        assert lib.mgv_oracle_f2h(float(f)) == h
    rng = np.random.Generator(np.random.Philox(1))
    vals = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s
                           for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 7e4)])
    vals = np.concatenate([vals, np.array([65504, 65519.9, 65520, 2.0 ** -24, 2.0 ** -25,
                                           1.5 * 2.0 ** -25, 2049, 2051, 0.0, -0.0], np.float32)])
    want = vals.astype(np.float16).view(np.uint16)
    got = np.array([lib.mgv_oracle_f2h(float(v)) for v in vals], dtype=np.uint16)
    assert (got == want).all()


def test_preprocess_matches_reference_golden(golden):
    g = golden["preprocess"]
    names = _names(g, "__dst")
    assert len(names) >= 8
    for name in names:
        meta = g[name + "__meta"]
        shape, layout, qt = [int(v) for v in meta[:-2]], int(meta[-2]), int(meta[-1])
        got = oracle.preprocess_weights(g[name + "__src"], shape, layout, qt)
        assert np.array_equal(got, g[name + "__dst"]), name


def test_row_and_column_major_inputs_give_identical_output():
    rng = np.random.Generator(np.random.Philox(3))
    K, N = 128, 192
    w = rng.integers(-8, 8, size=(N, K), dtype=np.int8)          # (n, k)
    col = synth.pack_int4_np(w)                                   # element (k,n) at n*K+k
    row = synth.pack_int4_np(np.ascontiguousarray(w.T))           # element (k,n) at k*N+n
    a = oracle.preprocess_weights(col, (K, N), oracle.COLUMN_MAJOR, oracle.W4_A16)
    b = oracle.preprocess_weights(row, (K, N), oracle.ROW_MAJOR, oracle.W4_A16)
    assert np.array_equal(a, b)
    w8 = rng.integers(-128, 128, size=(N, K), dtype=np.int8)
    a = oracle.preprocess_weights(w8.view(np.uint8), (K, N), oracle.COLUMN_MAJOR, oracle.W8_A16)
    b = oracle.preprocess_weights(np.ascontiguousarray(w8.T).view(np.uint8), (K, N), oracle.ROW_MAJOR, oracle.W8_A16)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("bits", [4, 8])
def test_layout_closed_form_reads_back_every_weight(bits):
    rng = np.random.Generator(np.random.Philox(4))
    K, N = 64, 24
    lo, hi = (-8, 8) if bits == 4 else (-128, 128)
    w = rng.integers(lo, hi, size=(N, K), dtype=np.int8)
    src = synth.pack_int4_np(w) if bits == 4 else w.view(np.uint8)
    pre = oracle.preprocess_weights(src, (K, N), oracle.COLUMN_MAJOR, oracle.W4_A16 if bits == 4 else oracle.W8_A16)
    for n in range(N):
        for k in range(K):
            assert oracle.read_preprocessed(pre, N, K, bits, n, k) == int(w[n, k])


def test_preprocess_refuses_what_the_reference_exits_on():
    src = np.zeros(64 * 64 // 2, dtype=np.uint8)
    with pytest.raises(ValueError):
        oracle.preprocess_weights(src, (64, 64), oracle.COLUMN_MAJOR, oracle.W4_AFP8)
    with pytest.raises(ValueError):
        oracle.preprocess_weights(src[: 64 * 6 // 2], (64, 6), oracle.COLUMN_MAJOR, oracle.W4_A16)   # N % 4
    with pytest.raises(ValueError):
        oracle.preprocess_weights(src[: 60 * 8 // 2], (60, 8), oracle.COLUMN_MAJOR, oracle.W4_A16)   # K % 8
    with pytest.raises(ValueError):
        oracle.preprocess_weights(src[: 64 * 32 // 2], (64, 32), oracle.ROW_MAJOR, oracle.W4_A16)    # 32-byte rule
    with pytest.raises(ValueError):
        oracle.preprocess_weights(src, (4, 4, 4, 32), oracle.COLUMN_MAJOR, oracle.W4_A16)            # rank


def test_zero_and_pack_golden(golden):
    g = golden["misc"]
    assert np.array_equal(oracle.preprocess_zeros(g["zeros__scales"], g["zeros__zeros"]).view(np.uint16),
                          g["zeros__out"].view(np.uint16))
    assert np.array_equal(oracle.pack_int4(g["pack__unpacked"]), g["pack__packed"])
    assert np.array_equal(oracle.unpack_int4(g["pack__packed"]), g["pack__roundtrip"])
    assert np.array_equal(g["pack__roundtrip"], g["pack__unpacked"])          # mixed_gemv_test.cu:211-217
    assert np.array_equal(synth.pack_int4_np(g["pack__unpacked"]), g["pack__packed"])


def test_gemv_matches_reference_golden_bit_for_bit(golden):
    g = golden["gemv_int4"]
    names = _names(g, "__out")
    assert len(names) >= 4
    for name in names:
        N, K, group = [int(v) for v in g[name + "__meta"]]
        w = synth.pack_int4_np(g[name + "__w"])
        zero = g[name + "__zero_i8"] if name + "__zero_i8" in g.files else None
        bias = g[name + "__bias"] if name + "__bias" in g.files else None
        for threads in (1, 3):
            got = oracle.gemv(w, g[name + "__x"], g[name + "__scale"], bits=4, group_size=group,
                              zero=zero, bias=bias, n_threads=threads)
            assert np.array_equal(got.view(np.uint16).ravel(), g[name + "__out"].view(np.uint16)), name


def test_int8_zero_points_equal_preprocessed_fp16_zeros(golden):
    """host/mixed_gemv.h:92-93 and utils/preprocess.h:99 produce the same additive term."""
    g = golden["gemv_int4"]
    name = "g64_zeros_bias"
    N, K, group = [int(v) for v in g[name + "__meta"]]
    w = synth.pack_int4_np(g[name + "__w"])
    zf = oracle.preprocess_zeros(g[name + "__scale"], g[name + "__zero_i8"])
    got = oracle.gemv(w, g[name + "__x"], g[name + "__scale"], bits=4, group_size=group, zero=zf,
                      bias=g[name + "__bias"])
    assert np.array_equal(got.view(np.uint16).ravel(), g[name + "__out"].view(np.uint16))


@pytest.mark.skipif(not oracle.have_ref(), reason="reference shim not built on this machine")
def test_restatement_against_live_reference_on_fresh_seeds():
    for seed in range(3):
        c = synth.make_case(1, 96, 512, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=128,
                            zeros="int8", bias=True, seed=seed, scale_range=(0.1, 0.3))
        want = oracle.ref_host_gemv_int4(c.w, c.x[0], c.scale, c.zero_i8, c.bias, group_size=128, n_threads=2)
        got = oracle.gemv(c.w, c.x, c.scale, bits=4, group_size=128, zero=c.zero_i8, bias=c.bias)
        assert np.array_equal(got.view(np.uint16).ravel(), want.view(np.uint16))
        for layout in (oracle.COLUMN_MAJOR,):
            a = oracle.preprocess_weights(c.w, (c.K, c.N), layout, oracle.W4_A16)
            b = oracle.ref_preprocess_weights(c.w, (c.K, c.N), layout, oracle.W4_A16)
            assert np.array_equal(a, b)
    rng = np.random.Generator(np.random.Philox(9))
    w8 = rng.integers(-128, 128, size=(3, 96, 64), dtype=np.int8).view(np.uint8)
    for layout in (oracle.COLUMN_MAJOR, oracle.ROW_MAJOR):
        a = oracle.preprocess_weights(w8, (3, 96, 64), layout, oracle.W8_A16)
        b = oracle.ref_preprocess_weights(w8, (3, 96, 64), layout, oracle.W8_A16)
        assert np.array_equal(a, b)


def test_gemv_properties_linearity_and_batch_rows():
    c = synth.make_case(3, 40, 256, bits=8, quant_op=Q.PER_COLUMN_SCALE_ONLY, bias=True, seed=5,
                        scale_range=(0.001, 0.01))
    full, acc = oracle.gemv(c.w, c.x, c.scale, bits=8, group_size=c.K, bias=c.bias, want_f32=True)
    for m in range(3):   # a batch is the same GEMV once per activation row
        one = oracle.gemv(c.w, c.x[m], c.scale, bits=8, group_size=c.K, bias=c.bias)
        assert np.array_equal(one.view(np.uint16), full[m:m + 1].view(np.uint16))
    # exact integer check of the fp32 accumulator against a float64 evaluation of the same terms
    dq = (c.w_unpacked.astype(np.float32).astype(np.float16).astype(np.float32)
          * c.scale[0].astype(np.float32)[:, None]).astype(np.float16).astype(np.float64)
    want = c.x.astype(np.float64) @ dq.T
    assert np.abs(acc - want).max() < 1e-4
    # alpha/beta
    ab = oracle.gemv(c.w, c.x, c.scale, bits=8, group_size=c.K, bias=c.bias, alpha=0.5, beta=2.0)
    want_ab = (0.5 * acc + 2.0 * c.bias.astype(np.float32)[None, :]).astype(np.float16)
    assert np.array_equal(ab.view(np.uint16), want_ab.view(np.uint16))


def test_tolerance_rule():
    c = synth.config("c2_int4_g128", N=64, K=256)
    rtol, atol = synth.tolerance(c)
    assert rtol == 1e-2 and abs(atol - 1e-2 * 16 * float(c.scale.max())) < 1e-9
    want = np.linspace(-1, 1, 64, dtype=np.float32)
    ok, _, _ = synth.check_close(want.copy(), want, c)
    assert ok
    bad = want.copy()
    bad[3] += 2 * atol + 2 * rtol
    assert not synth.check_close(bad, want, c)[0]
