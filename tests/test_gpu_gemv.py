"""GPU parity of the GEMV kernels against the CPU checker, through the C ABI.

Tolerance (stated by the task): max relative error 1e-2 and max absolute error
1e-2*sqrt(K)*max|scale| -- synth.check_close.  The kernels round the dequantised weight at the
same two places as the reference, so the observed error is orders of magnitude below it; the
tests also assert that tighter, observed-behaviour bound (fp32 summation order is the only
difference): |err| <= 2 fp16 ulp of the output.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from mixed_gemv_b200 import api, synth
from mixed_gemv_b200.enums import Status, Variant, WeightOnlyQuantOp as Q
from mixed_gemv_b200 import _lib as L
from mixed_gemv_b200._lib import MgvError
from tests.gpu_util import DeviceCase, oracle_out

pytestmark = pytest.mark.gpu

SIMT, MMA = Variant.SIMT, Variant.MMA


def _assert_close(got, want, case, tight=True, exact_rounding=False):
    """The stated tolerance, then a tighter bound from the arithmetic itself: 2 fp16 ulp of the
    output plus a fraction of the largest output -- 1e-6 for the SIMT family (same rounding points
    as the reference, only the fp32 summation order differs), 5e-4 for the MMA family (it skips
    the reference's per-weight fp16 roundings, which perturbs a sum by about 2^-12 of its terms)."""
    ok, max_abs, max_rel = synth.check_close(got, want, case)
    assert ok, (case.name, max_abs, max_rel, synth.tolerance(case))
    if tight:
        w = np.abs(want.astype(np.float32))
        ulp = np.maximum(np.spacing(w.astype(np.float16)).astype(np.float32), 2.0 ** -24)
        slack = (1e-6 if exact_rounding else 5e-4) * w.max()
        err = np.abs(got.astype(np.float32) - want.astype(np.float32))
        assert (err <= 2 * ulp + slack).all(), (case.name, float((err - 2 * ulp).max()), slack)


def test_golden_vectors_of_the_reference_host_gemv(cuda_lib, golden):
    g = golden["gemv_int4"]
    for name in sorted(k[:-5] for k in g.files if k.endswith("__out")):
        N, K, group = [int(v) for v in g[name + "__meta"]]
        zi = g[name + "__zero_i8"] if name + "__zero_i8" in g.files else None
        bias = g[name + "__bias"] if name + "__bias" in g.files else None
        scale = g[name + "__scale"]
        op = Q.FINEGRAINED_SCALE_AND_ZEROS if zi is not None else (Q.PER_COLUMN_SCALE_ONLY if group == K else Q.FINEGRAINED_SCALE_ONLY)
        zero = None
        if zi is not None:   # the device takes -zero*scale in fp16, produced by the GPU zero-point kernel
            zt = torch.zeros(scale.shape, dtype=torch.float16, device="cuda")
            api.ZeroPointPreprocessor.neg_zero_point_multiplies_scale(
                zt, torch.from_numpy(scale.copy()).cuda(), torch.from_numpy(zi.copy()).cuda(), scale.size)
            zero = zt.cpu().numpy()
        c = synth.Case(M=1, N=N, K=K, bits=4, quant_op=op, group_size=group, w=synth.pack_int4_np(g[name + "__w"]),
                       w_unpacked=g[name + "__w"], x=g[name + "__x"][None, :], scale=scale, zero=zero, zero_i8=zi,
                       bias=bias, name=name)
        d = DeviceCase(c)
        for variant in (SIMT, MMA):
            _assert_close(d.run(variant=variant)[0], g[name + "__out"], c, exact_rounding=variant == SIMT)


MODES = [
    ("percol", dict(quant_op=Q.PER_COLUMN_SCALE_ONLY)),
    ("g128", dict(quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128)),
    ("g64z", dict(quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=64, zeros="f16")),
]
SHAPES = [(64, 64), (4, 64), (100, 128), (36, 1024), (256, 4096), (1000, 576), (2048, 512), (4736, 1088)]


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("mode", MODES, ids=[m[0] for m in MODES])
@pytest.mark.parametrize("variant", [SIMT, MMA], ids=["simt", "mma"])
def test_modes_bits_shapes_m1(cuda_lib, bits, mode, variant):
    for i, (N, K) in enumerate(SHAPES):
        if (bits == 8 and N % 2) or K % mode[1].get("group_size", K):
            continue
        c = synth.make_case(1, N, K, bits=bits, bias=(i % 2 == 0), seed=i, x_dist="normal" if i % 3 else "uniform",
                            name=f"{mode[0]}-{bits}-{N}x{K}", **mode[1])
        d = DeviceCase(c)
        _assert_close(d.run(variant=variant), oracle_out(c), c, exact_rounding=variant == SIMT)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [2, 3, 4, 5, 8, 9, 16])
def test_batch_rows(cuda_lib, bits, M):
    c = synth.make_case(M, 520, 1536, bits=bits, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=64, zeros="f16",
                        bias=True, x_dist="normal", seed=M)
    d = DeviceCase(c)
    want = oracle_out(c)
    _assert_close(d.run(variant=MMA), want, c)
    if M <= 4:
        _assert_close(d.run(variant=SIMT), want, c, exact_rounding=True)
    # AUTO must pick something valid for every M
    _assert_close(d.run(variant=Variant.AUTO), want, c)


@pytest.mark.parametrize("bits,group,zeros,N,K,M", [(4, 128, False, 4800, 4096, 16), (4, 64, True, 9536, 8192, 16), (4, 64, True, 4768, 2048, 9),
                                                    (4, 128, True, 148 * 32 * 3 + 32, 6144, 12), (4, 4096, False, 4736, 4096, 13),
                                                    (8, 128, True, 2384, 8192, 16), (8, 2048, False, 4752, 2048, 10), (8, 64, False, 1024, 6144, 16)])
def test_single_pass_batch_kernel(cuda_lib, bits, group, zeros, N, K, M):
    """Batches of 9..16 rows at K = 2048, 4096, 6144, 8192 run on the single-pass kernel (one launch,
    every weight byte read once); it must match the checker, repeat its bits, and agree with the
    general kernel.  The N values give thread blocks with odd and even numbers of tiles."""
    op = Q.FINEGRAINED_SCALE_AND_ZEROS if zeros else (Q.PER_COLUMN_SCALE_ONLY if group == K else Q.FINEGRAINED_SCALE_ONLY)
    c = synth.make_case(M, N, K, bits=bits, quant_op=op, group_size=group, zeros="f16", bias=True, x_dist="normal", seed=N % 79,
                        scale_range=(0.001, 0.02) if bits == 4 else (0.001, 0.01))
    d = DeviceCase(c)
    want = oracle_out(c)
    a = d.arguments(variant=MMA)
    run = api.GemvAdaptor()
    run.initialize(a)
    assert run.launch_info.stages == 2 and run.launch_info.block == 512      # the batch kernel's ring: one slot per tile of a group
    run.run()
    torch.cuda.synchronize()
    got = a.out.cpu().numpy()
    _assert_close(got, want, c)
    a.out.fill_(float("nan"))
    run.run()
    torch.cuda.synchronize()
    assert np.array_equal(got.view(np.uint16), a.out.cpu().numpy().view(np.uint16))
    _assert_close(d.run(variant=MMA, hints=L.HINT_KERNEL_GENERAL), want, c)
    assert api.device_error_state() == 0


FULL_SIZE = [(name, M) for name in synth.CONFIG_NAMES + ["ref_shape"] for M in ((1, 8, 16) if name.startswith("c3") else (1,))]


@pytest.mark.parametrize("name,M", FULL_SIZE, ids=[f"{n}-M{m}" for n, m in FULL_SIZE])
def test_benchmark_configs_at_full_size(cuda_lib, name, M):
    """Every benchmark configuration by name, at its full size, on a sample of at least 256 output
    rows against the CPU checker (the checker runs on the sampled rows only); both kernel families
    where the batch allows.  `ref_shape` is the one shape the reference's own driver runs
    (mixed_gemv_test.cu:84,187,191: N = 151936, K = 2048, groups of 128, int8 zero-points)."""
    c = synth.config(name, M=M, seed=5)
    d = DeviceCase(c)
    rows = np.unique(np.concatenate([np.arange(0, c.N, max(1, c.N // 300)), np.arange(c.N - 40, c.N)]))
    assert rows.size >= 256
    sub_w = c.w_unpacked[rows]
    want = oracle.gemv(synth.pack_int4_np(sub_w) if c.bits == 4 else np.ascontiguousarray(sub_w), c.x,
                       np.ascontiguousarray(c.scale[:, rows]), bits=c.bits, group_size=c.group_size,
                       zero=None if c.zero is None else np.ascontiguousarray(c.zero[:, rows]),
                       bias=None if c.bias is None else c.bias[rows], n_threads=oracle.max_threads())
    for variant in ((MMA, SIMT) if M <= 4 else (MMA,)):
        got = d.run(variant=variant)
        assert np.isfinite(got.astype(np.float32)).all()
        _assert_close(got[:, rows], want, c, exact_rounding=variant == SIMT)
    if name == "ref_shape" and oracle.have_ref():
        # the reference's own host GEMV, live, on the same sampled rows (int8 zero-points)
        ref = oracle.ref_host_gemv_int4(synth.pack_int4_np(sub_w), c.x[0], np.ascontiguousarray(c.scale[:, rows]),
                                        np.ascontiguousarray(c.zero_i8[:, rows]), None, group_size=c.group_size,
                                        n_threads=oracle.max_threads())
        assert np.array_equal(np.asarray(ref).view(np.uint16).ravel(), want.view(np.uint16).ravel())


@pytest.mark.parametrize("group", [64, 128, 256, 512, 1024, 2048])
def test_group_sizes(cuda_lib, group):
    c = synth.make_case(1, 132, 2048, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=group, zeros="f16", seed=group)
    d = DeviceCase(c)
    for variant in (SIMT, MMA):
        _assert_close(d.run(variant=variant), oracle_out(c), c)


def test_with_and_without_split_k_scratch_agree(cuda_lib):
    """K-heavy, N-small shape: tiles are split over blocks when scratch is given, whole tiles per
    block when it is not; both must match the checker, and repeated calls must reuse the scratch.
    HINT_DEAL_ITEMS makes the library cut tiles whenever scratch is there, whatever its estimate."""
    c = synth.make_case(2, 256, 11008, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128, x_dist="normal", seed=3)
    d = DeviceCase(c)
    want = oracle_out(c)
    for variant in (SIMT, MMA):
        a = d.arguments(variant=variant, hints=L.HINT_DEAL_ITEMS)
        assert a.workspace is not None
        op = api.GemvAdaptor()
        op.initialize(a)
        assert op.launch_info.split_tiles > 0
        for _ in range(3):       # the kernel must leave the scratch ready for the next launch
            a.out.fill_(float("nan"))
            op.run()
            torch.cuda.synchronize()
            _assert_close(a.out.cpu().numpy(), want, c)
        first = a.out.cpu().numpy().copy()
        op.run(); torch.cuda.synchronize()
        assert np.array_equal(first.view(np.uint16), a.out.cpu().numpy().view(np.uint16))   # deterministic
        _assert_close(d.run(variant=variant, workspace=None, hints=L.HINT_DEAL_ITEMS), want, c)
    assert api.device_error_state() == 0


@pytest.mark.parametrize("bits,N,K,M", [(4, 11008, 4096, 1), (4, 4736 + 96, 1088, 3), (8, 4096, 2048, 2), (4, 9504, 576, 1)])
def test_dealing_modes_agree(cuda_lib, bits, N, K, M):
    """Whole tiles per block, halved tile ranges per cluster of two blocks (combined through
    distributed shared memory) and equal item ranges (combined through scratch) must all match the
    checker; each one keeps a fixed summation order, so repeating a call repeats its bits."""
    c = synth.make_case(M, N, K, bits=bits, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=64, zeros="f16", bias=True,
                        x_dist="normal", seed=N % 97)
    d = DeviceCase(c)
    want = oracle_out(c)
    for mode in (L.HINT_DEAL_TILES, L.HINT_DEAL_PAIRS, L.HINT_DEAL_ITEMS):
        for variant in ((SIMT, MMA) if M <= 4 else (MMA,)):
            got = d.run(variant=variant, hints=mode)
            _assert_close(got, want, c, exact_rounding=variant == SIMT)
            again = d.run(variant=variant, hints=mode)
            assert np.array_equal(got.view(np.uint16), again.view(np.uint16)), (mode, variant)


def test_programmatic_dependent_launch_keeps_stream_order(cuda_lib):
    """MGV_FLAG_PDL lets a call start while the previous kernel drains.  A chain in which each
    GEMV consumes the previous one's output (out1 -> x2 -> out2 -> x3) must still give the chained
    result, repeatedly, and with a slow kernel (a large fill) right in front of it."""
    K1, N1, N2, N3 = 1024, 2048, 1024, 512
    c1 = synth.make_case(1, N1, K1, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128, seed=1, scale_range=(0.01, 0.03))
    c2 = synth.make_case(1, N2, N1, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128, seed=2, scale_range=(0.01, 0.03))
    c3 = synth.make_case(1, N3, N2, bits=8, quant_op=Q.PER_COLUMN_SCALE_ONLY, seed=3, scale_range=(0.001, 0.003))
    d1, d2, d3 = DeviceCase(c1), DeviceCase(c2), DeviceCase(c3)
    y1 = oracle.gemv(c1.w, c1.x, c1.scale, bits=4, group_size=128)
    y2 = oracle.gemv(c2.w, y1, c2.scale, bits=4, group_size=128)
    y3 = oracle.gemv(c3.w, y2, c3.scale, bits=8, group_size=N2)
    o1 = torch.zeros(1, N1, dtype=torch.float16, device="cuda")
    o2 = torch.zeros(1, N2, dtype=torch.float16, device="cuda")
    o3 = torch.zeros(1, N3, dtype=torch.float16, device="cuda")
    a1 = d1.arguments(out=o1, flags=8)
    d2.x = o1
    a2 = d2.arguments(out=o2, flags=8)
    d3.x = o2
    a3 = d3.arguments(out=o3, flags=8)
    ops = []
    for a in (a1, a2, a3):
        op = api.GemvAdaptor()
        op.initialize(a)
        ops.append(op)
    junk = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    for rep in range(5):
        o1.zero_(); o2.zero_(); o3.zero_()
        junk.fill_(rep)                      # a long kernel right before the chain
        for op in ops:
            op.run()
        torch.cuda.synchronize()
        # outputs feed the next GEMV, so small differences propagate: compare with the tolerance of each stage
        assert synth.check_close(o1.cpu().numpy(), y1, c1)[0]
        y2_dev = oracle.gemv(c2.w, o1.cpu().numpy(), c2.scale, bits=4, group_size=128)
        assert synth.check_close(o2.cpu().numpy(), y2_dev, c2)[0]
        y3_dev = oracle.gemv(c3.w, o2.cpu().numpy(), c3.scale, bits=8, group_size=N2)
        assert synth.check_close(o3.cpu().numpy(), y3_dev, c3)[0]
    assert np.isfinite(y3.astype(np.float32)).all()


@pytest.mark.parametrize("bits,group,zeros,N,K,M", [(4, 128, False, 2048, 4096, 1), (4, 128, True, 1000, 2048 + 128, 3),
                                                     (4, 256, True, 4736, 1024, 9), (8, 128, True, 2050, 1536, 2),
                                                     (4, 2048, False, 4100, 2048, 16), (8, 1024, False, 512, 1024, 1)])
def test_item_lengths_agree(cuda_lib, bits, group, zeros, N, K, M):
    """The MMA kernels exist for items of 128 and of 256 k (HINT_ITEM_* forces one); both must match
    the checker, including a K that is not a multiple of 256 and a group that is half an item."""
    op = Q.FINEGRAINED_SCALE_AND_ZEROS if zeros else (Q.PER_COLUMN_SCALE_ONLY if group == K else Q.FINEGRAINED_SCALE_ONLY)
    c = synth.make_case(M, N, K, bits=bits, quant_op=op, group_size=group, zeros="f16", bias=True, x_dist="normal", seed=K % 89)
    d = DeviceCase(c)
    want = oracle_out(c)
    for item, hint in ((128, L.HINT_ITEM_128), (256, L.HINT_ITEM_256)):
        a = d.arguments(variant=MMA, hints=hint)
        run = api.GemvAdaptor()
        run.initialize(a)
        assert run.launch_info.k_slice == item or (item == 256 and M == 16)   # 256 needs room in shared memory
        run.run()
        torch.cuda.synchronize()
        _assert_close(a.out.cpu().numpy(), want, c)


@pytest.mark.parametrize("bits,group,zeros,N,K,M", [(4, 128, False, 2080, 4096, 1), (4, 64, True, 1056, 4096, 3), (4, 64, True, 4736, 8192, 8),
                                                    (4, 128, True, 2048, 8192, 5), (4, 4096, False, 2048, 4096, 7), (4, 256, False, 11008, 4096, 1),
                                                    (8, 4096, False, 1040, 4096, 2), (8, 128, True, 2048, 8192, 8), (8, 64, False, 4096, 4096, 1),
                                                    (4, 128, True, 151936 // 16, 2048, 1), (4, 64, False, 3104, 2048, 6), (4, 128, False, 4800, 6144, 1),
                                                    (4, 64, True, 2048, 6144, 8), (8, 2048, False, 1024, 2048, 1), (8, 128, True, 1504, 6144, 4)])
def test_x_in_registers_agrees(cuda_lib, bits, group, zeros, N, K, M):
    """For K = 2048, 4096, 6144 and 8192 the steady-state kernel has a form that keeps each warp's
    x fragments in registers instead of staging x in shared memory (HINT_KERNEL_* forces one or
    the other); both forms must match the checker and repeat their bits."""
    op = Q.FINEGRAINED_SCALE_AND_ZEROS if zeros else (Q.PER_COLUMN_SCALE_ONLY if group == K else Q.FINEGRAINED_SCALE_ONLY)
    c = synth.make_case(M, N, K, bits=bits, quant_op=op, group_size=group, zeros="f16", bias=True, x_dist="normal", seed=N % 83,
                        scale_range=(0.001, 0.02) if bits == 4 else (0.001, 0.01))
    d = DeviceCase(c)
    want = oracle_out(c)
    for hint, block_kind in ((L.HINT_KERNEL_XREG, "x in registers"), (L.HINT_KERNEL_STAGED, "x staged")):
        a = d.arguments(variant=MMA, hints=hint)
        run = api.GemvAdaptor()
        run.initialize(a)
        run.run()
        torch.cuda.synchronize()
        got = a.out.cpu().numpy()
        _assert_close(got, want, c)
        a.out.fill_(float("nan"))
        run.run()
        torch.cuda.synchronize()
        assert np.array_equal(got.view(np.uint16), a.out.cpu().numpy().view(np.uint16))
    assert api.device_error_state() == 0


@pytest.mark.parametrize("bits,group,zeros,N,K,M", [(4, 128, False, 32 * 148 * 3, 4096, 1), (4, 64, True, 32 * 148 * 2, 8192, 4),
                                                    (4, 128, True, 32 * 148 * 4, 2048, 2), (8, 4096, False, 16 * 148 * 3, 4096, 1),
                                                    (4, 128, False, 32 * 148 * 5, 6144, 8)])
def test_first_ring_fill_by_bulk_copy_changes_no_bit(cuda_lib, bits, group, zeros, N, K, M):
    """A launch without MGV_FLAG_PDL fills its ring first by tiled bulk copies (a tensor map of the
    weights), a launch with the flag by per-lane copies; the arithmetic is the same, so the two
    outputs must agree bit for bit (and with the checker), over blocks of several tiles."""
    op = Q.FINEGRAINED_SCALE_AND_ZEROS if zeros else (Q.PER_COLUMN_SCALE_ONLY if group == K else Q.FINEGRAINED_SCALE_ONLY)
    c = synth.make_case(M, N, K, bits=bits, quant_op=op, group_size=group, zeros="f16", bias=True, x_dist="normal", seed=K % 89,
                        scale_range=(0.001, 0.02) if bits == 4 else (0.001, 0.01))
    d = DeviceCase(c)
    rows = np.arange(0, N, max(1, N // 512))
    outs = []
    for flags in (0, L.FLAG_PDL):
        a = d.arguments(variant=MMA, flags=flags, hints=L.HINT_KERNEL_XREG)
        api.GemvAdaptor()(a)
        torch.cuda.synchronize()
        outs.append(a.out.cpu().numpy())
    assert api.device_error_state() == 0
    assert np.array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16))
    sub_w = c.w_unpacked[rows]
    want = oracle.gemv(synth.pack_int4_np(sub_w) if bits == 4 else np.ascontiguousarray(sub_w), c.x, np.ascontiguousarray(c.scale[:, rows]),
                       bits=bits, group_size=c.group_size, zero=None if c.zero is None else np.ascontiguousarray(c.zero[:, rows]),
                       bias=c.bias[rows], n_threads=oracle.max_threads())
    sub = synth.Case(M=M, N=rows.size, K=K, bits=bits, quant_op=op, group_size=c.group_size, w=None, w_unpacked=sub_w, x=c.x,
                     scale=np.ascontiguousarray(c.scale[:, rows]), zero=None, zero_i8=None, bias=c.bias[rows])
    _assert_close(outs[0][:, rows], want, sub, tight=False)


@pytest.mark.parametrize("bits,op,group,N,K,M,variant", [(4, Q.FINEGRAINED_SCALE_ONLY, 128, 2048, 4096, 1, MMA),
                                                         (4, Q.FINEGRAINED_SCALE_AND_ZEROS, 64, 22016, 4096, 2, MMA),
                                                         (8, Q.PER_COLUMN_SCALE_ONLY, 2048, 1024, 2048, 3, MMA),
                                                         (4, Q.FINEGRAINED_SCALE_ONLY, 128, 1000, 1024, 2, MMA),
                                                         (4, Q.FINEGRAINED_SCALE_ONLY, 128, 1000, 1024, 2, SIMT),
                                                         (4, Q.FINEGRAINED_SCALE_AND_ZEROS, 128, 4096, 11008, 1, MMA)])
def test_gated_silu_epilogue(cuda_lib, bits, op, group, N, K, M, variant):
    """MGV_FLAG_GATED_SILU: rows 2i / 2i+1 are gate and up of feature i, out[m][i] = silu(g)*u, N/2 outputs."""
    c = synth.make_case(M, N, K, bits=bits, quant_op=op, group_size=group, zeros="f16", bias=True, x_dist="normal", seed=N % 61,
                        scale_range=(0.001, 0.02) if bits == 4 else (0.001, 0.01))
    d = DeviceCase(c)
    out = torch.full((M, N // 2), float("nan"), dtype=torch.float16, device="cuda")
    a = d.arguments(variant=variant, out=out, flags=16)
    a.ldd = N // 2
    api.GemvAdaptor()(a)
    torch.cuda.synchronize()
    _, acc = oracle_out(c, want_f32=True)                     # fp32 sums before bias and rounding
    r = acc.astype(np.float64) + c.bias.astype(np.float64)[None, :]
    g, u = r[:, 0::2], r[:, 1::2]
    want = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    got = out.cpu().numpy().astype(np.float32)
    assert np.all(np.isfinite(got))
    scale_top = float(np.abs(c.scale.astype(np.float32)).max())
    atol = 1e-2 * np.sqrt(K) * scale_top * (1.0 + float(np.abs(r).max()))   # the product of two outputs carries both errors
    assert np.all(np.abs(got - want) <= atol + 2e-2 * np.abs(want)), float(np.abs(got - want).max())
    assert float(np.abs(got - want).max()) <= 4e-3 * float(np.abs(want).max()) + 1e-3
    # refusals
    a.flags = 16 | 1
    with pytest.raises(MgvError):
        api.GemvAdaptor()(a)
    a.flags = 16 | 4
    with pytest.raises(MgvError):
        api.GemvAdaptor()(a)


@pytest.mark.parametrize("bits,group,zeros,N,K,M", [(4, 128, False, 32 * 148 * 8, 4096, 8),    # x in registers, 8 tiles per block, 6 park slots
                                                    (4, 128, True, 32 * 148 * 3, 2048, 4),     # x staged, 3 tiles per block, 2 park slots
                                                    (8, 2048, False, 16 * 148 * 5, 2048, 8),   # 8-bit, x staged, 5 tiles per block, 2 park slots
                                                    (4, 64, True, 32 * 148 * 13, 8192, 1)])    # 13 tiles per block, 8 park slots, two groups per item
def test_steady_state_kernels_over_several_rounds(cuda_lib, bits, group, zeros, N, K, M):
    """A block that owns more tiles than its shared-memory partial buffer has slots works in rounds;
    the steady-state kernels must carry their rings, cursors and accumulators across them."""
    op = Q.FINEGRAINED_SCALE_AND_ZEROS if zeros else (Q.PER_COLUMN_SCALE_ONLY if group == K else Q.FINEGRAINED_SCALE_ONLY)
    c = synth.make_case(M, N, K, bits=bits, quant_op=op, group_size=group, zeros="f16", bias=True, x_dist="normal", seed=7,
                        scale_range=(0.001, 0.02) if bits == 4 else (0.001, 0.01))
    d = DeviceCase(c)
    got = d.run(variant=MMA)
    _assert_close(got, oracle_out(c), c)


def test_alpha_beta_partial_and_activation(cuda_lib):
    c = synth.make_case(1, 260, 1024, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128, bias=True, seed=11)
    d = DeviceCase(c)
    want, acc = oracle_out(c, want_f32=True)
    for variant in (SIMT, MMA):
        got = d.run(variant=variant, alpha=0.5, beta=2.0)
        _assert_close(got, oracle_out(c, alpha=0.5, beta=2.0), c)
        part = d.run(variant=variant, flags=1)                      # fp32 partial, no bias, no rounding
        assert part.dtype == np.float32
        assert np.abs(part - acc).max() <= (1e-5 if variant == SIMT else 5e-4) * np.abs(acc).max() + 1e-6
        relu = d.run(variant=variant, flags=2)
        _assert_close(relu, np.maximum(want.astype(np.float32), 0).astype(np.float16), c)
        silu = d.run(variant=variant, flags=4)
        v = (acc + c.bias.astype(np.float32)[None, :]).astype(np.float64)
        _assert_close(silu, (v / (1 + np.exp(-v))).astype(np.float16), c, tight=False)


def test_leading_dimensions_and_batch_strides(cuda_lib):
    """The reference's batch_count/batch_stride_* path (gemv/kernel/mixed_gemv.h:134,146-149):
    three problems with their own weights, activations, scales and outputs in one launch."""
    B, M, N, K = 3, 2, 96, 640
    cases = [synth.make_case(M, N, K, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128, bias=True, seed=40 + b)
             for b in range(B)]
    devs = [DeviceCase(c) for c in cases]
    ldx, ldd = K + 64, N + 10
    w = torch.stack([d.w for d in devs]).contiguous()
    x = torch.zeros(B, M, ldx, dtype=torch.float16, device="cuda")
    for b, d in enumerate(devs):
        x[b, :, :K] = d.x
    scale = torch.stack([d.scale for d in devs]).contiguous()
    bias = torch.stack([d.bias for d in devs]).contiguous()
    out = torch.full((B, M, ldd), -7.0, dtype=torch.float16, device="cuda")
    a = api.Arguments(M=M, N=N, K=K, weights=w, x=x, scale=scale, out=out, bias=bias, weight_bits=4,
                      quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128, batch_count=B, ldx=ldx, ldd=ldd,
                      batch_stride_weights=N * K // 2, batch_stride_x=M * ldx, batch_stride_scale=scale[0].numel(),
                      batch_stride_bias=N, batch_stride_out=M * ldd)
    for variant in (SIMT, MMA):
        a.variant = variant
        a.workspace = api.GemvAdaptor.allocate_workspace(a)
        out.fill_(-7.0)
        api.GemvAdaptor()(a)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        for b, c in enumerate(cases):
            _assert_close(got[b, :, :N], oracle_out(c), c)
        assert (got[:, :, N:] == -7.0).all()          # padding beyond N untouched


def test_device_gemv_keeps_the_reference_argument_order(cuda_lib):
    c = synth.make_case(1, 128, 512, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=128, zeros="int8",
                        scale_range=(0.1, 0.3), seed=5)
    d = DeviceCase(c)
    out = torch.zeros(1, c.N, dtype=torch.float16, device="cuda")
    # device_gemv(ptr_A, ptr_B, ptr_scale, ptr_zero_point, ptr_C, ptr_D, B, M_ref, N_ref, K, group_size)
    api.device_gemv(d.w, d.x, d.scale, d.zero, None, out, 1, c.N, 1, c.K, 128)
    torch.cuda.synchronize()
    want = oracle.gemv(c.w, c.x, c.scale, bits=4, group_size=128, zero=c.zero_i8)     # int8 zero-points, as the reference
    _assert_close(out.cpu().numpy(), want, c)


def test_linearity_property_full_size(cuda_lib):
    """Size-independent property at a benchmark size: GEMV(x1 + x2) == GEMV(x1) + GEMV(x2) in the fp32
    partial output when x1 and x2 have disjoint support, and a row permutation of the weights
    permutes the outputs."""
    c = synth.config("c2_int4_g128")
    d = DeviceCase(c)
    x = c.x.copy()
    x1, x2 = x.copy(), x.copy()
    x1[:, c.K // 2:] = 0
    x2[:, :c.K // 2] = 0
    outs = []
    for xx in (x, x1, x2):
        d.x = torch.from_numpy(xx).cuda()
        outs.append(d.run(variant=MMA, flags=1).astype(np.float64))
    assert np.abs(outs[0] - (outs[1] + outs[2])).max() <= 1e-4 * np.abs(outs[0]).max()
    # a sample of rows against the checker at full K
    rows = np.arange(0, c.N, 97)
    sub = synth.Case(M=1, N=rows.size, K=c.K, bits=4, quant_op=c.quant_op, group_size=c.group_size,
                     w=synth.pack_int4_np(c.w_unpacked[rows]), w_unpacked=c.w_unpacked[rows], x=c.x,
                     scale=np.ascontiguousarray(c.scale[:, rows]), zero=None, zero_i8=None, bias=None)
    d.x = torch.from_numpy(x).cuda()
    for variant in (SIMT, MMA):
        got = d.run(variant=variant)
        _assert_close(got[:, rows], oracle_out(sub), sub)


def test_argument_validation_returns_statuses(cuda_lib):
    c = synth.make_case(1, 64, 128, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=64, seed=1)
    d = DeviceCase(c)

    def status_of(**changes):
        a = d.arguments()
        for k, v in changes.items():
            setattr(a, k, v)
        with pytest.raises(MgvError) as e:
            api.GemvAdaptor()(a)
        return e.value.status

    assert status_of(group_size=32) == Status.INVALID_ARGUMENT            # gemv_adaptor.h:199-203
    assert status_of(group_size=96) == Status.INVALID_ARGUMENT            # K % group
    assert status_of(M=17) == Status.INVALID_ARGUMENT
    assert status_of(M=0) == Status.INVALID_ARGUMENT
    assert status_of(N=66) == Status.INVALID_ARGUMENT                     # N % 4
    assert status_of(K=100) == Status.INVALID_ARGUMENT                    # K % 64
    assert status_of(weight_bits=5) == Status.INVALID_ARGUMENT
    assert status_of(quant_op=Q.UNDEFINED) == Status.INVALID_ARGUMENT
    assert status_of(ldx=c.K + 4) == Status.MISALIGNED
    assert status_of(variant=Variant.SIMT, M=8) in (Status.UNSUPPORTED, Status.INVALID_ARGUMENT)
    assert status_of(quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS) == Status.INVALID_ARGUMENT   # zero missing
    assert status_of(x=d.x.view(-1)[4:]) == Status.MISALIGNED             # 8 bytes off a 16-byte boundary
    # the library stays usable after refusals
    _assert_close(d.run(), oracle_out(c), c)


def test_resident_layer_host_buffers(cuda_lib):
    c = synth.make_case(4, 300, 768, bits=8, quant_op=Q.PER_COLUMN_SCALE_ONLY, bias=True, seed=8, scale_range=(0.001, 0.01))
    layer = api.Linear(c, max_M=4)
    x = torch.from_numpy(c.x.copy()).pin_memory()
    out = torch.zeros(4, c.N, dtype=torch.float16).pin_memory()
    for M in (1, 4):
        layer.forward_host(x, out, M=M)
        _assert_close(out[:M].numpy(), oracle_out(c, M=M), c)
    # pinned buffers replay a captured graph from the second call on: same buffers, new contents
    want4 = oracle_out(c, M=4)
    for k in range(3):
        out.zero_()
        layer.forward_host(x, out, M=4)
        _assert_close(out.numpy(), want4, c)
    x.mul_(0.5)
    out.zero_()
    layer.forward_host(x, out, M=4)
    c_half = synth.make_case(4, 300, 768, bits=8, quant_op=Q.PER_COLUMN_SCALE_ONLY, bias=True, seed=8, scale_range=(0.001, 0.01))
    c_half.x[:] = x.numpy()
    _assert_close(out.numpy(), oracle_out(c_half, M=4), c_half)
    out2 = torch.zeros(4, c.N, dtype=torch.float16).pin_memory()   # other buffers: the graph is rebuilt
    layer.forward_host(x, out2, M=2)
    _assert_close(out2[:2].numpy(), oracle_out(c_half, M=2), c_half)
    pageable = torch.zeros(1, c.N, dtype=torch.float16)
    layer.forward_host(torch.from_numpy(c.x[:1].copy()), pageable, M=1)
    _assert_close(pageable.numpy(), oracle_out(c, M=1), c)
    with pytest.raises(MgvError):
        layer.forward_host(x, out, M=5)
    layer.close()
