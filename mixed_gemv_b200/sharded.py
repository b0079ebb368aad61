"""Sharding one large quantised layer over the GPUs of a node (one process per GPU).

The reference is single-GPU; these are the two natural cuts of D[N] = W[N,K] . x[K]:

* column split (over N, output features): rows are independent.  Because the preprocessed
  layout is blocked by 4 (int4) or 2 (int8) rows, each holding 2K contiguous bytes, a rank's
  shard of the FULL preprocessed buffer is one contiguous byte range, and equals the
  preprocessed shard.  Scales, zeros and bias shard as column slices; x is replicated.
  One exchange step follows the kernel: an all-gather of the fp16 output slices.
* row split (over K, the reduction): each rank owns a K range on group boundaries, must
  preprocess ITS range as its own {K_r, N} matrix (a K slice of the full preprocessed buffer
  is strided), emits fp32 partial sums (MGV_FLAG_OUT_F32_PARTIAL), and an all-reduce of the
  partials is followed by bias + fp16 rounding once.

The planning functions are pure host arithmetic (tested on CPU with gloo ranks); the layer
classes launch the CUDA kernel and call torch.distributed (NCCL on GPUs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .enums import WeightOnlyQuantOp
from .exchange import COUNTERS_OFFSET, SEEN_OFFSET, STATE_OFFSET, common_grid, counter_offset, source_mask


class ShardError(ValueError):
    pass


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    begin: int   # first row (column split) or first k (row split)
    end: int

    @property
    def size(self) -> int:
        return self.end - self.begin


def plan_column_split(N: int, world: int, rank: int, align: int = 64) -> Shard:
    """Rows [begin, end) of rank `rank`; boundaries on multiples of `align` rows (a multiple of
    the 4-row interleave), remainder blocks going to the first ranks."""
    if world < 1 or not (0 <= rank < world):
        raise ShardError(f"bad rank {rank} of {world}")
    if align % 4 or N % align:
        raise ShardError(f"N={N} must be a multiple of the shard alignment {align} (itself a multiple of 4)")
    blocks = N // align
    if blocks < world:
        raise ShardError(f"N={N} has fewer than {world} blocks of {align} rows")
    base, rem = divmod(blocks, world)
    begin = (rank * base + min(rank, rem)) * align
    end = begin + (base + (1 if rank < rem else 0)) * align
    return Shard(rank, world, begin, end)


def plan_row_split(K: int, world: int, rank: int, group_size: int) -> Shard:
    """k range [begin, end) of rank `rank`; boundaries on multiples of lcm(group_size, 64)."""
    if world < 1 or not (0 <= rank < world):
        raise ShardError(f"bad rank {rank} of {world}")
    align = int(np.lcm(group_size, 64))
    if K % align:
        raise ShardError(f"K={K} must be a multiple of {align}")
    blocks = K // align
    if blocks < world:
        raise ShardError(f"K={K} has fewer than {world} blocks of {align}")
    base, rem = divmod(blocks, world)
    begin = (rank * base + min(rank, rem)) * align
    end = begin + (base + (1 if rank < rem else 0)) * align
    return Shard(rank, world, begin, end)


def column_shard_bytes(shard: Shard, K: int, bits: int) -> tuple[int, int]:
    """Byte range of the shard inside the full PREPROCESSED weight buffer."""
    return shard.begin * K * bits // 8, shard.end * K * bits // 8


def slice_case_columns(case, shard: Shard):
    """Host-side column shard of a synth.Case (un-preprocessed weights)."""
    from .synth import Case, pack_int4_np
    wu = case.w_unpacked[shard.begin:shard.end]
    w = pack_int4_np(wu) if case.bits == 4 else np.ascontiguousarray(wu)
    sl = lambda a: None if a is None else np.ascontiguousarray(a[..., shard.begin:shard.end])
    return Case(M=case.M, N=shard.size, K=case.K, bits=case.bits, quant_op=case.quant_op,
                group_size=case.group_size, w=w, w_unpacked=wu, x=case.x, scale=sl(case.scale),
                zero=sl(case.zero), zero_i8=sl(case.zero_i8), bias=sl(case.bias), name=case.name)


def slice_case_rows(case, shard: Shard):
    """Host-side K shard of a synth.Case: weights [:, k0:k1], x[:, k0:k1], scale groups of the range."""
    from .synth import Case, pack_int4_np
    if case.quant_op == WeightOnlyQuantOp.PER_COLUMN_SCALE_ONLY:
        g0, g1, group = 0, 1, shard.size
    else:
        g0, g1, group = shard.begin // case.group_size, shard.end // case.group_size, case.group_size
    wu = np.ascontiguousarray(case.w_unpacked[:, shard.begin:shard.end])
    w = pack_int4_np(wu) if case.bits == 4 else wu
    sg = lambda a: None if a is None else np.ascontiguousarray(a[g0:g1])
    return Case(M=case.M, N=case.N, K=shard.size, bits=case.bits, quant_op=case.quant_op, group_size=group,
                w=w, w_unpacked=wu, x=np.ascontiguousarray(case.x[:, shard.begin:shard.end]), scale=sg(case.scale),
                zero=sg(case.zero), zero_i8=sg(case.zero_i8), bias=case.bias, name=case.name)


@dataclass
class DeviceShard:
    """One rank's shard, resident on its GPU: PREPROCESSED weights and the operands that go with
    them.  The layer classes take either this (a caller that already holds its shard on the
    device: from_tensors) or a host-side synth.Case (tests and benches: from_case uploads and
    preprocesses it)."""
    N: int
    K: int
    bits: int
    quant_op: WeightOnlyQuantOp
    group_size: int
    w: torch.Tensor
    scale: torch.Tensor
    zero: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None

    @classmethod
    def from_tensors(cls, w_preprocessed: torch.Tensor, scale: torch.Tensor, *, N: int, K: int, bits: int = 4,
                     quant_op=WeightOnlyQuantOp.FINEGRAINED_SCALE_ONLY, group_size: int = 128,
                     zero: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> "DeviceShard":
        for name, ten in (("weights", w_preprocessed), ("scale", scale), ("zero", zero), ("bias", bias)):
            if ten is not None and not ten.is_cuda:
                raise ShardError(f"{name} must be a CUDA tensor")
        if w_preprocessed.numel() * w_preprocessed.element_size() != N * K * bits // 8:
            raise ShardError(f"the weight buffer does not hold N*K*bits/8 = {N * K * bits // 8} bytes")
        if WeightOnlyQuantOp(quant_op) == WeightOnlyQuantOp.PER_COLUMN_SCALE_ONLY:
            group_size = K
        return cls(N, K, bits, WeightOnlyQuantOp(quant_op), group_size, w_preprocessed, scale, zero, bias)

    @classmethod
    def from_case(cls, case) -> "DeviceShard":
        from . import api
        dev = torch.device("cuda", torch.cuda.current_device())
        raw = torch.from_numpy(np.ascontiguousarray(case.w).view(np.uint8).ravel().copy()).to(dev)
        w = torch.empty_like(raw)
        api.MixedGemvWeightPreprocessor.run(w, raw, (case.K, case.N), 1, 1 if case.bits == 4 else 0)
        up = lambda a: None if a is None else torch.from_numpy(a.copy()).to(dev)
        return cls(case.N, case.K, case.bits, case.quant_op, case.group_size, w, up(case.scale), up(case.zero), up(case.bias))


def _as_device_shard(local) -> DeviceShard:
    return local if isinstance(local, DeviceShard) else DeviceShard.from_case(local)


def _check_world(group) -> tuple[int, int]:
    if not dist.is_initialized():
        raise ShardError("torch.distributed is not initialised")
    return dist.get_rank(group), dist.get_world_size(group)


class ColumnParallelGemv:
    """N-split layer: local GEMV into this rank's slice of the gathered output, then ONE
    all-gather (in place: the kernel writes straight into its segment of the gather buffer)."""

    def __init__(self, local_case, N_total: int, shard: Shard, group=None, max_M: int = 1, variant=0):
        from . import api
        self.api, self.group, self.shard, self.N_total = api, group, shard, N_total
        self.world = shard.world
        c = self.case = _as_device_shard(local_case)
        if shard.size != c.N:
            raise ShardError(f"shard has {shard.size} rows, the local weights have {c.N}")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.w, self.scale, self.zero, self.bias = c.w, c.scale, c.zero, c.bias
        self.max_M = max_M
        # gather buffer [world][M][n_local]: rank r's segment is contiguous
        self.gathered = torch.zeros(self.world, max_M, c.N, dtype=torch.float16, device=dev)
        self.variant = variant
        self._args = {}

    def _arguments(self, x: torch.Tensor, M: int):
        key = (x.data_ptr(), M)
        if key not in self._args:
            c = self.case
            a = self.api.Arguments(M=M, N=c.N, K=c.K, weights=self.w, x=x, scale=self.scale, zero=self.zero,
                                   bias=self.bias, out=self.gathered[self.shard.rank], weight_bits=c.bits,
                                   quant_op=c.quant_op, group_size=c.group_size, variant=self.variant)
            a.workspace = self.api.GemvAdaptor.allocate_workspace(a)
            op = self.api.GemvAdaptor()
            op.initialize(a)
            self._args[key] = op
        return self._args[key]

    def local(self, x: torch.Tensor, M: int = 1) -> None:
        self._arguments(x, M).run()

    def exchange(self) -> torch.Tensor:
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1), self.gathered[self.shard.rank].reshape(-1),
                                        group=self.group)
        return self.gathered

    def forward(self, x: torch.Tensor, M: int = 1) -> torch.Tensor:
        """Returns the gather buffer [world, max_M, n_local]; output feature n of rank r's shard is
        gathered[r, m, n - shard_begin(r)]."""
        self.local(x, M)
        return self.exchange()


class FusedColumnParallelGemv:
    """N-split layer whose exchange is fused into the kernel: the epilogue stores this rank's
    output slice into EVERY rank's gather buffer (peer stores over NVLink) and counts its thread
    blocks in on the peers' arrival counters; forward() then enqueues a bounded wait for the
    peers' arrivals instead of a collective.  No NCCL call on the data path.

    Two gather buffers alternate by call: call i+2 overwrites what call i gathered.  That is
    safe when, as in a decoder, a rank's call i+1 reads (directly or through the kernels before
    it) what call i gathered: a rank that starts call i+2 has seen every slice of call i+1, so
    every peer has finished call i+1 and with it all reads of call i's buffer.  All ranks must
    make the same sequence of calls.

    chained=True moves the wait into the NEXT call's kernel: call i+1 does not read its x before
    the peers' slices of call i have landed (it counts its launches itself), so a chain of layers
    needs no kernel between them and dependent launches keep overlapping; forward(complete=False)
    then returns a buffer that is valid once the next call -- or finish() -- has run.  All calls
    of a chained layer must have the same M (the launches must have the same grid).
    """

    def __init__(self, local_case, N_total: int, shard: Shard, group=None, max_M: int = 1, variant=0, flags: int = 0,
                 chained: bool = False):
        from . import api, exchange, _lib
        self.api, self.group, self.shard, self.N_total = api, group, shard, N_total
        self.world, self.rank = shard.world, shard.rank
        c = self.case = _as_device_shard(local_case)
        if shard.size != c.N:
            raise ShardError(f"shard has {shard.size} rows, the local weights have {c.N}")
        if self.world - 1 > 8:
            raise ShardError("the fused exchange reaches at most 8 peers")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.w, self.scale, self.zero, self.bias = c.w, c.scale, c.zero, c.bias
        self.max_M, self.variant, self.flags = max_M, variant, flags
        # every rank must hold the same window layout: shards of equal size only
        sizes = [None] * self.world
        dist.all_gather_object(sizes, int(c.N), group=group)
        if len(set(sizes)) != 1:
            raise ShardError(f"the fused exchange needs shards of equal size, got {sizes}")
        self.layout = exchange.layout(self.world, max_M, c.N, buffers=2)
        self.window = exchange.Window(self.layout.total_bytes)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.window.handle, group=group)
        self.peers = {r: exchange.PeerWindow(h) for r, h in enumerate(handles) if r != self.rank}
        self.gathered = [self.window.tensor(self.layout.segment_offset(b, 0), (self.world, max_M, c.N))
                         for b in range(self.layout.buffers)]
        self._ops, self._grids, self.calls = {}, {}, 0
        self.chained, self._pending = chained, 0
        self._lib, self._check = _lib.load(), _lib.check
        dist.barrier(group=group)  # every window is mapped before anyone stores into it

    def _op(self, x: torch.Tensor, M: int, buf: int):
        key = (x.data_ptr(), M, buf)
        if key not in self._ops:
            c, lay = self.case, self.layout
            seg = lay.segment_offset(buf, self.rank)
            order = sorted(self.peers)
            a = self.api.Arguments(M=M, N=c.N, K=c.K, weights=self.w, x=x, scale=self.scale, zero=self.zero,
                                   bias=self.bias, out=self.gathered[buf][self.rank], weight_bits=c.bits,
                                   quant_op=c.quant_op, group_size=c.group_size, variant=self.variant,
                                   flags=self.flags,
                                   peer_out=tuple(self.peers[r].ptr + seg for r in order),
                                   peer_flag=tuple(self.peers[r].ptr + counter_offset(self.rank) for r in order))
            if M not in self._grids:
                # arrivals per call and source: one per thread block of that rank's launch
                grids = [None] * self.world
                info = self.api.GemvAdaptor()
                info.initialize(a)
                dist.all_gather_object(grids, int(info.launch_info.grid), group=self.group)
                try:
                    self._grids[M] = common_grid(grids)
                except ValueError as e:
                    raise ShardError(str(e))
            if self.chained and self.world > 1:
                a.wait_flag = self.window.ptr + COUNTERS_OFFSET
                a.wait_state = self.window.ptr + STATE_OFFSET
                a.wait_delta = self._grids[M]
                a.wait_sources = source_mask(self.world, self.rank)
            op = self.api.GemvAdaptor()
            op.initialize(a)
            self._ops[key] = op
        return self._ops[key]

    def prepare(self, x: torch.Tensor, M: int = 1) -> None:
        """Builds the launch arguments of both buffers (collective: exchanges the grid sizes).
        Call it once per (x, M) on every rank before capturing forward() into a CUDA graph."""
        for b in range(self.layout.buffers):
            self._op(x, M, b)

    def forward(self, x: torch.Tensor, M: int = 1, complete: bool = True) -> torch.Tensor:
        """Enqueues the GEMV (with its peer stores) and, with complete=True, the wait for the
        peers' slices; returns the gather buffer of this call, [world, max_M, n_local], valid in
        stream order after that wait (or, in a chained layer, after the next call)."""
        if self.chained and self._grids and M not in self._grids:
            raise ShardError("all calls of a chained layer must have the same M")
        buf = self.calls % self.layout.buffers
        self.calls += 1
        self._op(x, M, buf).run()
        self._pending += self._grids[M]
        if complete:
            self.finish()
        return self.gathered[buf]

    def finish(self) -> None:
        """Enqueues the bounded wait for every peer slice of the calls made since the last wait."""
        if self.world > 1 and self._pending:
            import ctypes as C
            stream = int(torch.cuda.current_stream().cuda_stream)
            self._check(self._lib.mgv_wait_arrivals(C.c_void_p(self.window.ptr + COUNTERS_OFFSET),
                                                    C.c_void_p(self.window.ptr + SEEN_OFFSET),
                                                    C.c_uint32(source_mask(self.world, self.rank)),
                                                    C.c_uint32(self._pending & 0xffffffff), C.c_void_p(stream)))
        self._pending = 0

    def close(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody unmaps while a peer may still store
        for p in self.peers.values():
            p.close()
        self.peers = {}
        self.gathered = []
        dist.barrier(group=self.group)
        self.window.close()


class FusedRowParallelGemv:
    """K-split layer whose exchange is fused into the kernel: every rank's kernel stores its fp32
    partial output into its slot of EVERY rank's window (peer stores) and counts its thread blocks
    in; each rank then waits (bounded) for the peers' counts and adds the `world` partials in rank
    order -- the same order on every rank, so all ranks hold bit-identical outputs -- with bias and
    the fp16 rounding applied once (mgv_reduce_partials).  No collective on the data path.
    Two sets of slots alternate by call, as in FusedColumnParallelGemv."""

    def __init__(self, local_case, shard: Shard, group=None, max_M: int = 1, variant=0):
        from . import api, exchange, _lib
        self.api, self.group, self.shard = api, group, shard
        self.world, self.rank = shard.world, shard.rank
        c = self.case = _as_device_shard(local_case)
        if shard.size != c.K:
            raise ShardError(f"shard has {shard.size} k values, the local weights have {c.K}")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.w, self.scale, self.zero, self.bias = c.w, c.scale, c.zero, c.bias
        self.max_M, self.variant = max_M, variant
        self.layout = exchange.partials_layout(self.world, max_M, c.N, buffers=2)
        self.window = exchange.Window(self.layout.total_bytes)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.window.handle, group=group)
        self.peers = {r: exchange.PeerWindow(h) for r, h in enumerate(handles) if r != self.rank}
        self.out = torch.zeros(max_M, c.N, dtype=torch.float16, device=dev)
        self._ops, self._grids, self.calls, self._state_M = {}, {}, 0, None
        self._lib, self._check = _lib.load(), _lib.check
        dist.barrier(group=group)

    def _op(self, x_local: torch.Tensor, M: int, buf: int):
        key = (x_local.data_ptr(), M, buf)
        if key not in self._ops:
            c, lay = self.case, self.layout
            off = lay.part_offset(buf, self.rank)
            order = sorted(self.peers)
            a = self.api.Arguments(M=M, N=c.N, K=c.K, weights=self.w, x=x_local, scale=self.scale, zero=self.zero,
                                   bias=None, out=self.window.tensor(off, (self.max_M, c.N), "float32"),
                                   weight_bits=c.bits, quant_op=c.quant_op, group_size=c.group_size,
                                   variant=self.variant, flags=1,
                                   peer_out=tuple(self.peers[r].ptr + off for r in order),
                                   peer_flag=tuple(self.peers[r].ptr + counter_offset(self.rank) for r in order))
            op = self.api.GemvAdaptor()
            op.initialize(a)
            self._ops[key] = op
            if M not in self._grids:
                grids = [None] * self.world
                dist.all_gather_object(grids, int(op.launch_info.grid), group=self.group)
                try:
                    self._grids[M] = common_grid(grids)
                except ValueError as e:
                    raise ShardError(str(e))
        return self._ops[key]

    def forward(self, x_local: torch.Tensor, M: int = 1) -> torch.Tensor:
        """x_local: this rank's K range of x, [M][K_r].  Returns the full output [max_M][N] (fp16),
        identical on every rank, valid in stream order."""
        import ctypes as C
        buf = self.calls % self.layout.buffers
        self.calls += 1
        self._op(x_local, M, buf).run()
        stream = C.c_void_p(int(torch.cuda.current_stream().cuda_stream))
        lay = self.layout
        if self._state_M is not None and M != self._state_M:
            raise ShardError("the launch counter of the fused wait counts launches of one batch size: keep M fixed per layer object")
        self._state_M = M
        # one launch: every block waits (bounded) for this round's arrivals from all peers, then adds its share
        self._check(self._lib.mgv_wait_reduce_partials(
            C.c_void_p(self.window.ptr + lay.part_offset(buf, 0)), C.c_size_t(lay.part_bytes // 4), self.world, M, self.case.N,
            C.c_longlong(self.case.N), C.c_void_p(self.bias.data_ptr() if self.bias is not None else None), C.c_float(1.0), 0,
            C.c_void_p(self.out.data_ptr()), C.c_longlong(self.case.N),
            C.c_void_p(self.window.ptr + COUNTERS_OFFSET), C.c_void_p(self.window.ptr + STATE_OFFSET),
            C.c_uint32(source_mask(self.world, self.rank)), C.c_uint32(self._grids[M]), stream))
        return self.out

    def close(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for p in self.peers.values():
            p.close()
        self.peers = {}
        self._ops = {}
        dist.barrier(group=self.group)
        self.window.close()


class RowParallelGemv:
    """K-split layer: local GEMV to fp32 partials, all-reduce, then bias + fp16 rounding once."""

    def __init__(self, local_case, shard: Shard, group=None, max_M: int = 1, variant=0):
        from . import api
        self.api, self.group, self.shard = api, group, shard
        c = self.case = _as_device_shard(local_case)
        if shard.size != c.K:
            raise ShardError(f"shard has {shard.size} k values, the local weights have {c.K}")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.w, self.scale, self.zero, self.bias = c.w, c.scale, c.zero, c.bias
        self.partial = torch.zeros(max_M, c.N, dtype=torch.float32, device=dev)
        self.out = torch.zeros(max_M, c.N, dtype=torch.float16, device=dev)
        self.variant = variant
        self._args = {}

    def local(self, x_local: torch.Tensor, M: int = 1) -> None:
        key = (x_local.data_ptr(), M)
        if key not in self._args:
            c = self.case
            a = self.api.Arguments(M=M, N=c.N, K=c.K, weights=self.w, x=x_local, scale=self.scale, zero=self.zero,
                                   bias=None, out=self.partial, weight_bits=c.bits, quant_op=c.quant_op,
                                   group_size=c.group_size, variant=self.variant, flags=1)
            a.workspace = self.api.GemvAdaptor.allocate_workspace(a)
            op = self.api.GemvAdaptor()
            op.initialize(a)
            self._args[key] = op
        self._args[key].run()

    def exchange(self, M: int = 1) -> torch.Tensor:
        if self.shard.world > 1:
            dist.all_reduce(self.partial, op=dist.ReduceOp.SUM, group=self.group)
        import ctypes as C
        from . import _lib
        c = self.case
        _lib.check(_lib.load().mgv_reduce_partials(
            C.c_void_p(self.partial.data_ptr()), C.c_size_t(0), 1, M, c.N, C.c_longlong(c.N),
            C.c_void_p(self.bias.data_ptr() if self.bias is not None else None), C.c_float(1.0), 0,
            C.c_void_p(self.out.data_ptr()), C.c_longlong(c.N), C.c_void_p(int(torch.cuda.current_stream().cuda_stream))))
        return self.out             # bias added and rounded to fp16 once, after the reduction

    def forward(self, x_local: torch.Tensor, M: int = 1) -> torch.Tensor:
        self.local(x_local, M)
        return self.exchange(M)
