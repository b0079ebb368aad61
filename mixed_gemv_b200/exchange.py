"""Memory windows for the fused output exchange of an N-split layer (host plumbing).

A Window is device memory of this process's GPU that the other processes of the node can map
(CUDA IPC through the library's mgv_window_* entry points).  Its layout, shared by all ranks:

    [32 s, 32 s + 4)  arrival counter of SOURCE rank s (s = 0..8): that rank's thread blocks add 1
                      when their outputs have landed here.  One counter per source: with a single
                      summed counter a peer that runs a call ahead could stand in for another
                      peer's arrival that is still in flight.
    [320, 324)        arrivals per source already consumed by this rank's wait kernels
    [328, 336)        launches of this rank that waited inside the kernel so far
    [512, ...)        `buffers` gather buffers of world * max_M * n_local fp16 each (256-byte aligned)

`layout()` is pure arithmetic (tested on CPU); the classes need a GPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

COUNTER_STRIDE = 32       # MGV_COUNTER_STRIDE
COUNTERS_OFFSET = 0
SEEN_OFFSET = 320
STATE_OFFSET = 328
HEADER_BYTES = 512
HANDLE_BYTES = 64
MAX_WORLD = 9             # this rank and at most 8 peers


def counter_offset(source_rank: int) -> int:
    """Byte offset, in EVERY rank's window, of the counter that rank `source_rank` counts in on."""
    if not (0 <= source_rank < MAX_WORLD):
        raise ValueError(f"source rank {source_rank} outside 0..{MAX_WORLD - 1}")
    return COUNTERS_OFFSET + COUNTER_STRIDE * source_rank


def source_mask(world: int, rank: int) -> int:
    """Bit s set for every rank s != rank: the sources whose counters rank `rank` waits on."""
    if not (1 <= world <= MAX_WORLD and 0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    return sum(1 << s for s in range(world) if s != rank)


def common_grid(grids) -> int:
    """The one grid all ranks launch (the in-kernel wait counts `grid` arrivals per source and
    round); raises when the ranks' launches differ."""
    g = {int(v) for v in grids}
    if len(g) != 1:
        raise ValueError(f"the fused exchange needs the same launch grid on every rank, got {sorted(g)}")
    return g.pop()


def arrivals_ready(counters, sources: int, target: int) -> bool:
    """The waiter's test, as the kernels make it: every counter s with bit s of `sources` set has
    reached `target` (modulo 2^32: counters only grow)."""
    return all(((int(counters[s]) - target) & 0xffffffff) < 0x80000000
               for s in range(MAX_WORLD) if (sources >> s) & 1)


def wait_target(tickets_before: int, grid: int, delta: int, own_round: bool) -> int:
    """The arrivals a block must see from EACH source, as the kernels compute it from the launch
    counter: `tickets_before` blocks have drawn a ticket before this one, `grid` blocks make a
    launch.  The GEMV's in-kernel wait (own_round False) needs the rounds of the launches BEFORE
    its own; mgv_wait_reduce_partials (own_round True) also needs the round its own launch closes."""
    launch = tickets_before // grid
    return ((launch + (1 if own_round else 0)) * delta) & 0xffffffff


@dataclass(frozen=True)
class WindowLayout:
    world: int
    max_M: int
    n_local: int
    buffers: int

    @property
    def buffer_bytes(self) -> int:
        raw = self.world * self.max_M * self.n_local * 2
        return (raw + 255) // 256 * 256

    @property
    def total_bytes(self) -> int:
        return HEADER_BYTES + self.buffers * self.buffer_bytes

    def segment_offset(self, buffer: int, rank: int) -> int:
        """Byte offset of rank `rank`'s [max_M][n_local] segment inside gather buffer `buffer`."""
        if not (0 <= buffer < self.buffers and 0 <= rank < self.world):
            raise ValueError(f"buffer {buffer} / rank {rank} outside the window")
        return HEADER_BYTES + buffer * self.buffer_bytes + rank * self.max_M * self.n_local * 2


@dataclass(frozen=True)
class PartialsLayout:
    """Window of a K-split layer: `buffers` sets of `world` fp32 partial outputs [max_M][N]."""
    world: int
    max_M: int
    N: int
    buffers: int

    @property
    def part_bytes(self) -> int:
        return (self.max_M * self.N * 4 + 255) // 256 * 256

    @property
    def total_bytes(self) -> int:
        return HEADER_BYTES + self.buffers * self.world * self.part_bytes

    def part_offset(self, buffer: int, rank: int) -> int:
        """Byte offset of the partial output of rank `rank` inside set `buffer`."""
        if not (0 <= buffer < self.buffers and 0 <= rank < self.world):
            raise ValueError(f"buffer {buffer} / rank {rank} outside the window")
        return HEADER_BYTES + (buffer * self.world + rank) * self.part_bytes


def partials_layout(world: int, max_M: int, N: int, buffers: int = 2) -> PartialsLayout:
    if world < 1 or world > 8 + 1:
        raise ValueError("the fused exchange reaches at most 8 peers")
    if max_M < 1 or N < 1 or buffers < 1:
        raise ValueError("bad window shape")
    return PartialsLayout(world, max_M, N, buffers)


def layout(world: int, max_M: int, n_local: int, buffers: int = 2) -> WindowLayout:
    if world < 1 or world > 8 + 1:
        raise ValueError("the fused exchange reaches at most 8 peers")
    if max_M < 1 or n_local < 1 or buffers < 1:
        raise ValueError("bad window shape")
    return WindowLayout(world, max_M, n_local, buffers)


class _CudaView:
    """Minimal __cuda_array_interface__ carrier so torch can view window memory without copying."""

    def __init__(self, ptr: int, shape, typestr: str, owner):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}
        self._owner = owner


class Window:
    """This rank's window: owns the memory, exports the handle, views it as torch tensors."""

    def __init__(self, nbytes: int):
        from . import _lib
        self._lib = _lib.load()
        p = C.c_void_p()
        h = (C.c_ubyte * HANDLE_BYTES)()
        _lib.check(self._lib.mgv_window_create(C.byref(p), C.c_size_t(nbytes), h))
        self.ptr, self.nbytes, self.handle = int(p.value), nbytes, bytes(h)

    def tensor(self, offset: int, shape, dtype="float16"):
        import torch
        typestr = {"float16": "<f2", "float32": "<f4", "uint32": "<u4", "uint8": "|u1"}[dtype]
        n = int(np.prod(shape)) * int(typestr[2:])
        if offset < 0 or offset + n > self.nbytes:
            raise ValueError("view outside the window")
        return torch.as_tensor(_CudaView(self.ptr + offset, shape, typestr, self), device="cuda")

    def close(self) -> None:
        if self.ptr:
            self._lib.mgv_window_destroy(C.c_void_p(self.ptr))
            self.ptr = 0


class PeerWindow:
    """Another rank's window mapped into this process."""

    def __init__(self, handle: bytes):
        from . import _lib
        if len(handle) != HANDLE_BYTES:
            raise ValueError("an inter-process handle is 64 bytes")
        self._lib = _lib.load()
        p = C.c_void_p()
        buf = (C.c_ubyte * HANDLE_BYTES).from_buffer_copy(handle)
        _lib.check(self._lib.mgv_window_open(buf, C.byref(p)))
        self.ptr = int(p.value)

    def close(self) -> None:
        if self.ptr:
            self._lib.mgv_window_close(C.c_void_p(self.ptr))
            self.ptr = 0
