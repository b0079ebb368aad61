"""CPU tests of the fused output exchange's host logic: the window layout, the arrival arithmetic,
and the protocol itself run by world_size-2 and -3 gloo ranks over POSIX shared memory standing in for
the peer-mapped windows (the CPU checker stands in for the kernel, a byte-wise store for the
epilogue's peer stores, an integer add for the arrival count).  The failure case is injected on
the host: a rank that never stores makes the other rank's bounded wait give up with a status
instead of hanging."""
import os
import socket
import time
from multiprocessing import shared_memory

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from mixed_gemv_b200 import exchange, sharded, synth
from mixed_gemv_b200.enums import WeightOnlyQuantOp as Q


def test_window_layout():
    lay = exchange.layout(world=4, max_M=2, n_local=2752, buffers=2)
    seg = 2 * 2752 * 2
    assert lay.buffer_bytes % 256 == 0 and lay.buffer_bytes >= 4 * seg
    assert lay.total_bytes == exchange.HEADER_BYTES + 2 * lay.buffer_bytes
    assert lay.segment_offset(0, 0) == exchange.HEADER_BYTES
    assert lay.segment_offset(0, 3) == exchange.HEADER_BYTES + 3 * seg
    assert lay.segment_offset(1, 0) == exchange.HEADER_BYTES + lay.buffer_bytes
    offs = sorted(lay.segment_offset(b, r) for b in range(2) for r in range(4))
    assert all(b - a >= seg for a, b in zip(offs, offs[1:]))          # segments never overlap
    assert offs[-1] + seg <= lay.total_bytes
    offs = [exchange.counter_offset(s) for s in range(exchange.MAX_WORLD)]
    assert all(o % 4 == 0 for o in offs) and all(b - a == exchange.COUNTER_STRIDE for a, b in zip(offs, offs[1:]))
    assert offs[-1] + 4 <= exchange.SEEN_OFFSET and exchange.SEEN_OFFSET % 4 == 0 and exchange.STATE_OFFSET % 8 == 0
    assert exchange.SEEN_OFFSET + 4 <= exchange.STATE_OFFSET and exchange.STATE_OFFSET + 8 <= exchange.HEADER_BYTES
    for bad in ((0, 1, 64, 2), (10, 1, 64, 2), (2, 0, 64, 2), (2, 1, 0, 2), (2, 1, 64, 0)):
        with pytest.raises(ValueError):
            exchange.layout(*bad)
    with pytest.raises(ValueError):
        lay.segment_offset(2, 0)
    with pytest.raises(ValueError):
        lay.segment_offset(0, 4)


def test_partials_layout():
    lay = exchange.partials_layout(world=4, max_M=2, N=8192, buffers=2)
    assert lay.part_bytes == 2 * 8192 * 4 and lay.total_bytes == exchange.HEADER_BYTES + 2 * 4 * lay.part_bytes
    offs = sorted(lay.part_offset(b, r) for b in range(2) for r in range(4))
    assert offs[0] == exchange.HEADER_BYTES and all(b - a == lay.part_bytes for a, b in zip(offs, offs[1:]))
    assert offs[-1] + lay.part_bytes == lay.total_bytes
    assert lay.part_offset(1, 0) - lay.part_offset(0, 0) == 4 * lay.part_bytes     # the slots of a set are contiguous
    with pytest.raises(ValueError):
        lay.part_offset(0, 4)
    with pytest.raises(ValueError):
        exchange.partials_layout(2, 1, 0)


def test_sources_and_grids():
    assert exchange.source_mask(2, 0) == 0b10 and exchange.source_mask(4, 2) == 0b1011 and exchange.source_mask(1, 0) == 0
    assert exchange.common_grid([148, 148, 148]) == 148
    with pytest.raises(ValueError):
        exchange.common_grid([148, 128])
    with pytest.raises(ValueError):
        exchange.source_mask(10, 0)


def test_a_peer_running_ahead_cannot_stand_in_for_a_late_arrival():
    """Three ranks, grid g.  Rank A waits for round 1 of B and C.  B has finished round 1 AND,
    running a call ahead, round 2; C's last thread block of round 1 has not counted in yet.
    A single summed counter would read 2g + (g-1) >= 2g and let A through with C's slice
    incomplete; per-source counters keep A waiting until C's count arrives."""
    g = 5
    counters = np.zeros(exchange.MAX_WORLD, dtype=np.uint32)
    A, B, C_ = 0, 1, 2
    counters[B], counters[C_] = 2 * g, g - 1
    mask = exchange.source_mask(3, A)
    assert int(counters[B]) + int(counters[C_]) >= 2 * g               # the summed test would pass ...
    assert not exchange.arrivals_ready(counters, mask, g)              # ... the per-source test does not
    counters[C_] += 1                                                  # the withheld arrival lands
    assert exchange.arrivals_ready(counters, mask, g)
    assert not exchange.arrivals_ready(counters, mask, 2 * g)          # round 2: C has not started
    # counters only grow and are compared modulo 2^32
    counters[B], counters[C_] = 3, 0xfffffffe
    assert not exchange.arrivals_ready(counters, mask, 2)
    counters[C_] = (int(counters[C_]) + 4) & 0xffffffff
    assert exchange.arrivals_ready(counters, mask, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _counters(win):
    """The per-source counters of a window as a strided uint32 view."""
    words = np.ndarray((exchange.HEADER_BYTES // 4,), dtype=np.uint32, buffer=win.buf)
    return words[exchange.COUNTERS_OFFSET // 4::exchange.COUNTER_STRIDE // 4][:exchange.MAX_WORLD]


def _wait_arrivals(win, sources, delta, limit_s):
    """The wait kernel's logic: target = seen + delta, seen moves on, bounded polling of every source."""
    words = np.ndarray((exchange.HEADER_BYTES // 4,), dtype=np.uint32, buffer=win.buf)
    target = (int(words[exchange.SEEN_OFFSET // 4]) + delta) & 0xffffffff
    words[exchange.SEEN_OFFSET // 4] = target
    t0 = time.time()
    while not exchange.arrivals_ready(_counters(win), sources, target):
        if time.time() - t0 > limit_s:
            return False
        time.sleep(0.001)
    return True


def _rank_main(rank, world, port, silent_rank, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    wins, own = [], None
    try:
        c = synth.make_case(2, 384, 1024, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=128, zeros="f16",
                            bias=True, x_dist="normal", seed=11)
        sh = sharded.plan_column_split(c.N, world, rank)
        local = sharded.slice_case_columns(c, sh)
        lay = exchange.layout(world, c.M, local.N, buffers=2)
        own = shared_memory.SharedMemory(create=True, size=lay.total_bytes)
        own.buf[:lay.total_bytes] = bytes(lay.total_bytes)
        names = [None] * world
        dist.all_gather_object(names, own.name)
        wins = [own if r == rank else shared_memory.SharedMemory(name=n) for r, n in enumerate(names)]
        grids = [None] * world
        dist.all_gather_object(grids, 3)
        delta = exchange.common_grid(grids)                        # arrivals per source and call
        sources = exchange.source_mask(world, rank)
        dist.barrier()
        ok_all = True
        for call in range(4):                                      # both buffers, twice
            buf = call % lay.buffers
            x = (c.x * (call + 1)).astype(np.float16)
            if rank != silent_rank:
                y = oracle.gemv(local.w, x, local.scale, bits=4, group_size=128, zero=local.zero, bias=local.bias)
                seg = lay.segment_offset(buf, rank)
                for r, w in enumerate(wins):                       # "peer stores": every rank's buffer gets the slice
                    w.buf[seg:seg + y.nbytes] = y.tobytes()
                for r, w in enumerate(wins):                       # "arrival counts", one per thread block, on MY counter there
                    if r != rank:
                        cnt = _counters(w)
                        for _ in range(grids[rank]):
                            cnt[rank] = (int(cnt[rank]) + 1) & 0xffffffff
            ok = _wait_arrivals(own, sources, delta, limit_s=1.0 if (silent_rank >= 0 and rank != silent_rank) else 30.0)
            ok_all = ok_all and ok
            if ok and rank != silent_rank:                          # (a silent rank holds no slice of its own)
                g = np.ndarray((world, c.M, local.N), dtype=np.float16, buffer=own.buf,
                               offset=lay.segment_offset(buf, 0)).copy()
                got = np.concatenate([g[r] for r in range(world)], axis=1)
                want = oracle.gemv(c.w, x, c.scale, bits=4, group_size=128, zero=c.zero, bias=c.bias)
                assert np.array_equal(got.view(np.uint16), want.view(np.uint16))   # rows are independent: bit-exact
        tag = "ok" if ok_all else "timeout"
        open(os.path.join(out_dir, f"{tag}_{rank}"), "w").write(tag)
        dist.barrier()
    finally:
        for r, w in enumerate(wins):
            w.close()
        if own is not None:
            own.unlink()
        dist.destroy_process_group()


def test_two_gloo_ranks_exchange_through_windows(tmp_path):
    mp.spawn(_rank_main, args=(2, _free_port(), -1, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok_0", "ok_1"]


def test_three_gloo_ranks_exchange_through_windows(tmp_path):
    mp.spawn(_rank_main, args=(3, _free_port(), -1, str(tmp_path)), nprocs=3, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok_0", "ok_1", "ok_2"]


def test_a_silent_peer_ends_the_wait_with_a_status_not_a_hang(tmp_path):
    """Rank 1 never stores nor counts in (failure injected on the host); rank 0's bounded waits give
    up and report, rank 1 itself still receives rank 0's slices."""
    t0 = time.time()
    mp.spawn(_rank_main, args=(2, _free_port(), 1, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok_1", "timeout_0"]
    assert time.time() - t0 < 60


def test_launch_counter_gives_the_round_to_wait_for():
    """Blocks of successive launches draw tickets from one counter; the ticket tells a block which
    round of arrivals its launch needs, whichever order the blocks of a launch arrive in."""
    from mixed_gemv_b200 import exchange
    grid, delta = 148, 148
    for launch in range(4):
        for ticket in (launch * grid, launch * grid + 77, (launch + 1) * grid - 1):
            assert exchange.wait_target(ticket, grid, delta, own_round=False) == launch * delta
            assert exchange.wait_target(ticket, grid, delta, own_round=True) == (launch + 1) * delta
    # the wait-and-reduce launch of round 3 must not pass on the counts of rounds 1 and 2
    counters = [0] * exchange.MAX_WORLD
    counters[1] = 2 * delta
    need = exchange.wait_target(2 * 32 + 5, 32, delta, own_round=True)     # third launch of a 32-block grid
    assert need == 3 * delta and not exchange.arrivals_ready(counters, 0b10, need)
    counters[1] = 3 * delta
    assert exchange.arrivals_ready(counters, 0b10, need)
    # counters wrap modulo 2^32
    assert exchange.wait_target((2 ** 32 // delta + 1) * grid, grid, delta, own_round=False) == ((2 ** 32 // delta + 1) * delta) & 0xffffffff
