"""The fused output exchange on ONE GPU: the epilogue's extra stores and arrival counts with the
"peers" standing in as ordinary buffers of the same GPU, the wait that consumes the counts, and
the wait's time-out path (a counter nothing increments; the kernel gives up after about a
second, raises the error word and returns -- no fault, the context stays usable)."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

from tests.gpu_util import DeviceCase, oracle_out

pytestmark = pytest.mark.gpu


def _wait(lib, flag, seen, delta, sources=1):
    """`flag` is the counter of source 0 (bit 0 of `sources`); further sources sit 32 bytes apart behind it."""
    from mixed_gemv_b200 import _lib
    _lib.check(lib.mgv_wait_arrivals(C.c_void_p(flag.data_ptr()), C.c_void_p(seen.data_ptr()), C.c_uint32(sources), C.c_uint32(delta),
                                     C.c_void_p(int(torch.cuda.current_stream().cuda_stream))))


@pytest.mark.parametrize("name,M", [("c2_int4_g128", 1), ("c1_int8_percol_bias", 2), ("c3_int4_g64_zeros_bias", 1)])
def test_epilogue_stores_to_every_destination_and_counts_blocks(cuda_lib, name, M):
    from mixed_gemv_b200 import api, synth
    c = synth.config(name, M=M, N=2048, K=2048)
    d = DeviceCase(c)
    out = torch.zeros(M, c.N, dtype=torch.float16, device="cuda")
    peers = [torch.zeros_like(out) for _ in range(3)]
    flags = torch.zeros(3, 64, dtype=torch.int32, device="cuda")  # one counter per "peer", a cache line apart
    a = d.arguments(M=M, out=out)
    a.peer_out = tuple(p.data_ptr() for p in peers)
    a.peer_flag = (flags[0].data_ptr(), 0, flags[2].data_ptr())  # the second destination wants no signal
    op = api.GemvAdaptor()
    op.initialize(a)
    for _ in range(3):
        op.run()
    seen = torch.zeros(1, dtype=torch.int32, device="cuda")
    _wait(cuda_lib, flags[0], seen, 3 * op.launch_info.grid)  # producers ran earlier on this GPU
    torch.cuda.synchronize()
    want = oracle_out(c, M=M)
    assert synth.check_close(out.cpu().numpy(), want, c)[0]
    for p in peers:
        assert torch.equal(p, out)
    counts = flags[:, 0].cpu().numpy()
    assert counts[0] == counts[2] == 3 * op.launch_info.grid and counts[1] == 0
    assert int(seen.item()) == 3 * op.launch_info.grid
    assert api.device_error_state() == 0


def test_general_kernel_path_also_signals(cuda_lib):
    from mixed_gemv_b200 import api, synth, _lib
    c = synth.config("c2_int4_g128", N=1024, K=1024)
    d = DeviceCase(c)
    out = torch.zeros(1, c.N, dtype=torch.float16, device="cuda")
    peer = torch.zeros_like(out)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = d.arguments(out=out, hints=_lib.HINT_KERNEL_GENERAL)
    a.peer_out, a.peer_flag = (peer.data_ptr(),), (flag.data_ptr(),)
    op = api.GemvAdaptor()
    op.initialize(a)
    op.run()
    torch.cuda.synchronize()
    assert torch.equal(peer, out) and int(flag.item()) == op.launch_info.grid


def test_wait_gives_up_and_reports(cuda_lib):
    from mixed_gemv_b200 import api
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    seen = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    _wait(cuda_lib, flag, seen, 1)  # nothing will ever arrive
    state = api.device_error_state()  # synchronises
    assert 0.5 < time.time() - t0 < 10.0
    assert state == 0x20
    assert api.device_error_state() == 0  # read and cleared
    # the context is intact: ordinary work still runs
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0


def test_wait_inside_the_kernel_counts_its_launches(cuda_lib):
    """Launch L of a chain waits for L * delta arrivals: with the counter pre-set to what three
    earlier launches' peers would have delivered, four launches run through; the kernel's own
    launch count ends at 4 * grid."""
    from mixed_gemv_b200 import api, synth
    c = synth.config("c2_int4_g128", N=2048, K=2048)
    d = DeviceCase(c)
    out = torch.zeros(1, c.N, dtype=torch.float16, device="cuda")
    hdr = torch.zeros(64, dtype=torch.int32, device="cuda")  # [0]: arrival counter, [2:4]: launch counter (8 bytes)
    a = d.arguments(out=out, flags=8)
    a.wait_flag, a.wait_state, a.wait_delta, a.wait_sources = hdr.data_ptr(), hdr.data_ptr() + 8, 5, 1
    hdr[0] = 3 * 5
    op = api.GemvAdaptor()
    op.initialize(a)
    for _ in range(4):
        op.run()
    torch.cuda.synchronize()
    assert api.device_error_state() == 0
    assert int(hdr[2].item()) == 4 * op.launch_info.grid
    assert synth.check_close(out.cpu().numpy(), oracle_out(c), c)[0]


def test_partials_go_to_peers_and_reduce(cuda_lib):
    """K-split form on one GPU: the fp32 partials land in every destination; mgv_reduce_partials adds
    the slots in order and applies bias and the fp16 rounding once."""
    from mixed_gemv_b200 import _lib, api, synth
    c = synth.config("c3_int4_g64_zeros_bias", M=2, N=1024, K=2048)
    d = DeviceCase(c)
    slots = torch.zeros(3, 2, c.N, dtype=torch.float32, device="cuda")   # stand-ins for three ranks' slots
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = d.arguments(M=2, out=slots[0], flags=1)
    a.peer_out = (slots[1].data_ptr(), slots[2].data_ptr())
    a.peer_flag = (flag.data_ptr(), 0)
    op = api.GemvAdaptor()
    op.initialize(a)
    op.run()
    out = torch.zeros(2, c.N, dtype=torch.float16, device="cuda")
    stream = C.c_void_p(int(torch.cuda.current_stream().cuda_stream))
    _lib.check(cuda_lib.mgv_reduce_partials(C.c_void_p(slots.data_ptr()), C.c_size_t(2 * c.N), 3, 2, c.N, C.c_longlong(c.N),
                                            C.c_void_p(d.bias.data_ptr()), C.c_float(1.0), 0, C.c_void_p(out.data_ptr()),
                                            C.c_longlong(c.N), stream))
    torch.cuda.synchronize()
    assert torch.equal(slots[0], slots[1]) and torch.equal(slots[0], slots[2])
    assert int(flag.item()) == op.launch_info.grid
    _, acc = oracle_out(c, M=2, want_f32=True)                           # fp32 result before bias and rounding
    want = (3.0 * acc + c.bias.astype(np.float32)[None, :]).astype(np.float16)
    got = out.cpu().numpy()
    tol = 3 * 1e-2 * np.sqrt(c.K) * float(np.abs(c.scale.astype(np.float32)).max())
    assert np.all(np.abs(got.astype(np.float32) - want.astype(np.float32)) <= tol + 1e-2 * np.abs(want.astype(np.float32)))
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 2e-3 * np.abs(want.astype(np.float32)).max()


def test_wait_and_reduce_in_one_launch(cuda_lib):
    """mgv_wait_reduce_partials = mgv_wait_arrivals + mgv_reduce_partials: on one GPU, with local
    buffers as the peers' slots and a local counter as source 1, two rounds in a row give the same
    bits as the two-call form; a counter nothing increments makes the bounded wait give up after
    about a second with the error word set, and the context stays usable."""
    from mixed_gemv_b200 import _lib, api, synth
    c = synth.config("c3_int4_g64_zeros_bias", M=2, N=1024, K=2048)
    d = DeviceCase(c)
    slots = torch.zeros(3, 2, c.N, dtype=torch.float32, device="cuda")
    hdr = torch.zeros(128, dtype=torch.int32, device="cuda")          # counters 32 bytes apart, then the launch counter
    counters, state = hdr.data_ptr(), hdr.data_ptr() + 328
    a = d.arguments(M=2, out=slots[0], flags=1)
    a.peer_out = (slots[1].data_ptr(), slots[2].data_ptr())
    a.peer_flag = (counters + 32, 0)                                   # the kernel counts in as source 1
    op = api.GemvAdaptor()
    op.initialize(a)
    grid = op.launch_info.grid
    want = torch.zeros(2, c.N, dtype=torch.float16, device="cuda")
    got = torch.zeros(2, c.N, dtype=torch.float16, device="cuda")
    stream = C.c_void_p(int(torch.cuda.current_stream().cuda_stream))
    for rnd in range(2):
        op.run()
        got.zero_()
        _lib.check(cuda_lib.mgv_wait_reduce_partials(C.c_void_p(slots.data_ptr()), C.c_size_t(2 * c.N), 3, 2, c.N, C.c_longlong(c.N),
                                                     C.c_void_p(d.bias.data_ptr()), C.c_float(1.0), 8 if rnd else 0,
                                                     C.c_void_p(got.data_ptr()), C.c_longlong(c.N), C.c_void_p(counters),
                                                     C.c_void_p(state), C.c_uint32(0b10), C.c_uint32(grid), stream))
        _lib.check(cuda_lib.mgv_reduce_partials(C.c_void_p(slots.data_ptr()), C.c_size_t(2 * c.N), 3, 2, c.N, C.c_longlong(c.N),
                                                C.c_void_p(d.bias.data_ptr()), C.c_float(1.0), 0, C.c_void_p(want.data_ptr()),
                                                C.c_longlong(c.N), stream))
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert int(hdr[8].item()) == (rnd + 1) * grid
    assert api.device_error_state() == 0
    # a third round that nobody delivers: source 2 never counts in
    t0 = time.perf_counter()
    _lib.check(cuda_lib.mgv_wait_reduce_partials(C.c_void_p(slots.data_ptr()), C.c_size_t(2 * c.N), 3, 2, c.N, C.c_longlong(c.N),
                                                 C.c_void_p(d.bias.data_ptr()), C.c_float(1.0), 0, C.c_void_p(got.data_ptr()),
                                                 C.c_longlong(c.N), C.c_void_p(counters), C.c_void_p(state), C.c_uint32(0b100),
                                                 C.c_uint32(grid), stream))
    torch.cuda.synchronize()
    assert 0.5 < time.perf_counter() - t0 < 10.0
    assert api.device_error_state() & 0x20
    assert api.device_error_state() == 0                               # read and cleared, and the context still works
    op.run()
    torch.cuda.synchronize()
