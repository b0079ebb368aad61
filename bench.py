#!/usr/bin/env python
"""Benchmark of the weight-only-quantised GEMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--variant auto|simt|mma] [--M m] [--sets R]

The workload is a chain of GEMV calls over R distinct resident layers of the workload's shape
(R*bytes is several times the L2, so every call streams its weights from HBM).  A CUDA graph holds
several passes over the R layers; one STEP replays it often enough to last at least 50 ms.
`value` is algorithmic GB/s over the whole job (bytes each call must move, every operand counted
once, times calls, divided by device time); `ms_per_step` is the mean step, `ms_per_step_median`
the median; `us_per_call` is the per-launch figure the metric is quoted in; `isolated_us_per_call`
is the same chain without programmatic dependent launch (every kernel starts after its
predecessor has finished -- the figure comparable with a profiler's per-kernel duration).

N > 1 (one process per GPU under torchrun): an N-split layer whose per-GPU shard has the
workload's shape (weak scaling).  Every call delivers its output slice to all GPUs: by default
the kernel's epilogue stores it into the peers' gather buffers and a bounded wait kernel
consumes the peers' arrival counts (--exchange fused); --exchange nccl runs an NCCL all-gather
after every call instead, the baseline the fused path is measured against.
--split k cuts the layer over K instead: fp32 partials are exchanged (fused or NCCL all-reduce) and added, every
GPU ends with the full output.

`e2e` is the same metric through the host-buffer C ABI call (mgv_linear_forward_host): per call
the activations go host->device from pinned memory, the GEMV runs, the result comes back
device->host and the call waits for it.  Weights stay resident, as in the reference's own
driver (mixed_gemv_test.cu:264-283).

`--impl reference` times the reference's host GEMV (host/mixed_gemv.h:82-104; compiled from the
reference's headers when available, else the C restatement) on all host threads, one full call
of the same shape per step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DEFAULT_WORKLOAD = "c2_int4_g128"
METRIC = "achieved HBM GB/s of the int4 g128 M=1 GEMV (us/call in us_per_call)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--split", choices=["n", "k"], default="n",
                    help="N > 1: cut the layer over output features (n: every GPU holds a workload-shaped shard of the "
                         "rows and the output slices are exchanged) or over the reduction (k: every GPU holds a "
                         "workload-shaped shard of K, fp32 partials are exchanged and added)")
    ap.add_argument("--exchange", choices=["fused", "nccl", "none"], default="fused",
                    help="N > 1: how the output slices reach the other GPUs -- stored by the kernel's epilogue into "
                         "peer windows (fused) or by an NCCL all-gather after every call (nccl)")
    ap.add_argument("--variant", default="auto", choices=["auto", "simt", "mma"])
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--sets", type=int, default=0, help="distinct resident layers per step (0: >= 3x L2)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch (MGV_FLAG_PDL)")
    ap.add_argument("--prefetch-next", action="store_true",
                    help="give every call the next layer's weights as its prefetch hint (mgv_gemv_args.prefetch)")
    ap.add_argument("--no-workspace", action="store_true", help="give the kernel no split-K scratch (blocks own whole tiles)")
    ap.add_argument("--N", type=int, default=0, help="override the workload's N")
    ap.add_argument("--K", type=int, default=0, help="override the workload's K")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="N > 1: skip the strong-scaled 70B-class layers reported beside the weak-scaling headline")
    return ap.parse_args()


_KEEP = []   # graphs, windows and operators of finished measurements: never destructed before the process leaves


def init_dist(dev):
    import torch.distributed as dist
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)


def finish():
    """All ranks leave together, past their last collective, without unwinding the communicator
    (graphs that captured collectives are still alive; their destructor order hung here)."""
    import torch
    sys.stdout.flush()
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def workload_string(case):
    """The same text in the library's and the reference's lines (the shape every GPU works on)."""
    return f"{case.name}: M={case.M} K={case.K} N={case.N} group={case.group_size} per GPU"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback 6.65 TB/s (MEASURED_PEAKS.json absent)"


# DRAM bytes of ONE launch (dram__bytes_read.sum + dram__bytes_write.sum) from an ncu capture of the
# kernel the library picks for the shape; None for shapes that were not captured.  It cannot be
# measured by this script (a number taken under a profiler is not a bench value), so it is a
# recorded constant, labelled as such in the line.
CAPTURED_TRAFFIC = {
    ("c2_int4_g128", 1, 11008, 4096): (23334656, "gemv_tile_kernel<4,false,false,2,2,false>"),
}


def traffic_bytes(case):
    return CAPTURED_TRAFFIC.get((case.name, case.M, case.N, case.K), (None, None))


# --------------------------------------------------------------------------- CPU reference arm

def cpu_gemv_timing(case, repeats=1, threads=None):
    """Times the reference host GEMV on `threads` host threads (default: all); returns
    (seconds per call, kind, threads).  threads=1 is the reference as written: its host GEMV has
    no threading (host/mixed_gemv.h:82-104)."""
    from oracle import oracle
    import numpy as np
    threads = threads or max(1, os.cpu_count() or 1)
    # the reference's own host code handles int4 weights with int8 (or no) zero-points at M=1
    use_ref = (oracle.have_ref() and case.bits == 4 and case.M == 1
               and (case.zero is None or case.zero_i8 is not None))
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        if use_ref:
            oracle.ref_host_gemv_int4(case.w, case.x[0], case.scale, case.zero_i8, case.bias,
                                      group_size=case.group_size, n_threads=threads)
        else:
            oracle.gemv(case.w, case.x, case.scale, bits=case.bits, group_size=case.group_size,
                        zero=case.zero, bias=case.bias, n_threads=min(threads, oracle.max_threads()))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    if not use_ref:
        threads = min(threads, oracle.max_threads())
    return best, ("reference" if use_ref else "port"), threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mixed_gemv_b200 import synth
    case = synth.config(args.workload, M=args.M, seed=0)
    nbytes = case.algorithmic_bytes()
    kind = threads = None
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_gemv_timing(case)
    times = []
    for _ in range(args.steps):
        dt, kind, threads = cpu_gemv_timing(case)
        times.append(dt)
    total = sum(times)
    value = nbytes * len(times) / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "us_per_call": 1e6 * total / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 x int%d -> f32 accumulate" % case.bits, "data": "synthetic",
        "config": {"workload": workload_string(case), "step": "one full host GEMV call"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind,
                         "sample": "the full shape, one call per step, rows split over all host threads"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- clocks sampler

class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- our arm

def run_ours_ksplit(args):
    """N > 1, --split k: a layer cut over K.  Every rank holds a workload-shaped K shard (weak scaling: K_total =
    K * n_gpus), emits fp32 partials, and every rank ends with the full fp16 output: either the kernels store their
    partials into every GPU's window and a reduce kernel adds them in rank order after a bounded wait (fused), or
    an NCCL all-reduce adds them (nccl); bias and the fp16 rounding once, at the end."""
    import ctypes as C
    import numpy as np
    import torch
    import torch.distributed as dist
    from mixed_gemv_b200 import _lib, api, exchange, synth
    from mixed_gemv_b200.enums import LayoutType, QuantType, Variant
    from oracle import oracle

    world, rank, local_rank = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", "0"))
    api.require_cuda()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    init_dist(dev)
    lib = _lib.load()
    case = synth.config(args.workload, M=args.M, seed=rank, N=args.N or None, K=args.K or None)   # this rank's K shard
    bias_np = synth.config(args.workload, M=args.M, seed=0, N=args.N or None, K=args.K or None).bias  # one bias for the layer
    nbytes = case.algorithmic_bytes()
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    R = args.sets or max(8, -(-3 * l2 // nbytes))
    gen = torch.Generator(device=dev)
    gen.manual_seed(4321 + rank)
    raw0 = torch.from_numpy(np.ascontiguousarray(case.w).view(np.uint8).ravel().copy()).to(dev)
    weights = [torch.empty_like(raw0)]
    api.MixedGemvWeightPreprocessor.run(weights[0], raw0, (case.K, case.N), LayoutType.kColumnMajor,
                                        QuantType.W4_A16 if case.bits == 4 else QuantType.W8_A16)
    up = lambda a: None if a is None else torch.from_numpy(a.copy()).to(dev)
    scales, zeros = [up(case.scale)], [up(case.zero)]
    lo, hi = float(case.scale.min()), float(case.scale.max())
    for _ in range(1, R):
        weights.append(torch.randint(0, 256, raw0.shape, dtype=torch.uint8, device=dev, generator=gen))
        scales.append((torch.rand(case.scale.shape, device=dev, generator=gen) * (hi - lo) + lo).half())
        zeros.append(None if case.zero is None else (torch.rand(case.zero.shape, device=dev, generator=gen) * 0.1 - 0.05).half())
    x, bias = up(case.x), up(bias_np)
    fused = args.exchange == "fused"
    kernel_only = args.exchange == "none"      # no exchange at all: what the GEMV kernels alone take
    final = torch.zeros(R, case.M, case.N, dtype=torch.float16, device=dev)
    window, peers, lay, parts = None, {}, None, None
    if fused:
        lay = exchange.partials_layout(world, case.M, case.N, buffers=R)
        window = exchange.Window(lay.total_bytes)
        handles = [None] * world
        dist.all_gather_object(handles, window.handle)
        peers = {r: exchange.PeerWindow(h) for r, h in enumerate(handles) if r != rank}
        dist.barrier()
    else:
        parts = torch.zeros(R, case.M, case.N, dtype=torch.float32, device=dev)
    ops, arrivals = [], 0
    for r in range(R):
        out = window.tensor(lay.part_offset(r, rank), (case.M, case.N), "float32") if fused else parts[r]
        a = api.Arguments(M=case.M, N=case.N, K=case.K, weights=weights[r], x=x, scale=scales[r], zero=zeros[r], bias=None,
                          out=out, weight_bits=case.bits, quant_op=case.quant_op, group_size=case.group_size,
                          variant=Variant.MMA, flags=1 | (0 if args.no_pdl else 8))
        if fused:
            order = sorted(peers)
            a.peer_out = tuple(peers[q].ptr + lay.part_offset(r, rank) for q in order)
            a.peer_flag = tuple(peers[q].ptr + exchange.counter_offset(rank) for q in order)
        op = api.GemvAdaptor()
        op.initialize(a)
        ops.append(op)
    info = ops[0].launch_info
    arrivals = info.grid                      # per source and call: one per thread block of that rank's launch
    sources = exchange.source_mask(world, rank)

    def one_step():
        st = C.c_void_p(int(torch.cuda.current_stream().cuda_stream))
        for r in range(R):
            ops[r].run()
            if kernel_only:
                continue
            if fused:   # wait for the round's arrivals and add the partials in one launch
                _lib.check(lib.mgv_wait_reduce_partials(
                    C.c_void_p(window.ptr + lay.part_offset(r, 0)), C.c_size_t(lay.part_bytes // 4), world, case.M, case.N,
                    C.c_longlong(case.N), C.c_void_p(bias.data_ptr() if bias is not None else None), C.c_float(1.0),
                    0 if args.no_pdl else 8, C.c_void_p(final[r].data_ptr()), C.c_longlong(case.N),
                    C.c_void_p(window.ptr + exchange.COUNTERS_OFFSET), C.c_void_p(window.ptr + exchange.STATE_OFFSET),
                    C.c_uint32(sources), C.c_uint32(arrivals), st))
                continue
            dist.all_reduce(parts[r])
            src, stride, n_parts = parts[r].data_ptr(), 0, 1
            _lib.check(lib.mgv_reduce_partials(C.c_void_p(src), C.c_size_t(stride), n_parts, case.M, case.N, C.c_longlong(case.N),
                                               C.c_void_p(bias.data_ptr() if bias is not None else None), C.c_float(1.0), 0,
                                               C.c_void_p(final[r].data_ptr()), C.c_longlong(case.N), st))

    one_step()
    torch.cuda.synchronize()
    if api.device_error_state() != 0:
        raise RuntimeError("a device-side wait timed out")
    # check set 0 on a row sample: the ranks' fp32 partial sums of the CPU checker, added, plus bias
    rows = np.arange(0, case.N, max(1, case.N // 256))
    sub_w = case.w_unpacked[rows]
    _, acc = oracle.gemv(synth.pack_int4_np(sub_w) if case.bits == 4 else np.ascontiguousarray(sub_w), case.x,
                         np.ascontiguousarray(case.scale[:, rows]), bits=case.bits, group_size=case.group_size,
                         zero=None if case.zero is None else np.ascontiguousarray(case.zero[:, rows]), bias=None,
                         want_f32=True, n_threads=oracle.max_threads())
    tot = torch.from_numpy(acc.astype(np.float32)).to(dev)
    dist.all_reduce(tot)
    want = tot.cpu().numpy() + (0.0 if bias_np is None else bias_np.astype(np.float32)[rows][None, :])
    got = final[0].cpu().numpy()[:, rows].astype(np.float32)
    tol = 1e-2 * np.sqrt(case.K * world) * float(np.abs(case.scale.astype(np.float32)).max())
    max_abs = float(np.abs(got - want).max())
    if not kernel_only and not np.all(np.abs(got - want) <= tol + 1e-2 * np.abs(want)):
        raise RuntimeError(f"K-split output differs from the CPU checker: max_abs={max_abs}")

    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        one_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        one_step()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        graph.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(4):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    est = torch.tensor([e0.elapsed_time(e1) / 4], device=dev)
    dist.all_reduce(est, op=dist.ReduceOp.MAX)
    reps = max(1, int(20.0 / max(float(est.item()), 1e-4)))     # a step lasts at least 20 ms
    barrier()
    e0.record()
    for _ in range(args.steps * reps):
        graph.replay()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    calls = args.steps * reps * R
    peak, peak_src = peaks()
    value = world * nbytes * calls / (ms * 1e-3) / 1e9
    _KEEP.extend([graph, ops, window, peers, parts, final, weights, scales, zeros])
    how = ("the kernels themselves (peer stores + arrival counts, bounded wait, partials added in rank order)" if fused
           else "nothing (kernels only, no exchange)" if kernel_only else "an NCCL all-reduce")
    return {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms / args.steps, "us_per_call": 1e3 * ms / calls, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 x int%d -> f32 accumulate" % case.bits, "data": "synthetic",
        "config": {"workload": workload_string(case),
                   "sharding": f"K-split layer of K={case.K * world}, fp32 partials exchanged by " + how
                               + ", then bias and fp16 rounding once",
                   "calls_per_step": R, "grid": info.grid, "block": info.block, "stages": info.stages, "cuda_graph": True,
                   "programmatic_dependent_launch": not args.no_pdl,
                   "check": None if kernel_only else {"rows": int(rows.size), "max_abs": max_abs}},
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s", "frac": value / world / peak,
                     "traffic": None, "peak_source": peak_src, "bytes_per_launch": nbytes},
        "e2e": None, "cpu_baseline": None, "gpu_launches": calls * (1 if kernel_only else 3 if fused else 2), "clocks": None}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import ctypes as C
    from mixed_gemv_b200 import _lib, api, exchange, synth, sharded
    from mixed_gemv_b200.enums import LayoutType, QuantType, Variant

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    api.require_cuda()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    init_dist(dev)
    variant = {"auto": Variant.AUTO, "simt": Variant.SIMT, "mma": Variant.MMA}[args.variant]

    case = synth.config(args.workload, M=args.M, seed=rank, N=args.N or None, K=args.K or None)  # this rank's shard has the workload's shape
    nbytes = case.algorithmic_bytes()
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    R = args.sets or max(8, -(-3 * l2 // nbytes))
    qt = QuantType.W4_A16 if case.bits == 4 else QuantType.W8_A16

    # ---- resident layers: set 0 holds the seeded case (checked), the others random bytes ----
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    raw0 = torch.from_numpy(np.ascontiguousarray(case.w).view(np.uint8).ravel().copy()).to(dev)
    weights = [torch.empty_like(raw0)]
    api.MixedGemvWeightPreprocessor.run(weights[0], raw0, (case.K, case.N), LayoutType.kColumnMajor, qt)
    up = lambda a: None if a is None else torch.from_numpy(a.copy()).to(dev)
    scales, zeros = [up(case.scale)], [up(case.zero)]
    lo, hi = float(case.scale.min()), float(case.scale.max())
    for _ in range(1, R):
        weights.append(torch.randint(0, 256, raw0.shape, dtype=torch.uint8, device=dev, generator=gen))
        scales.append((torch.rand(case.scale.shape, device=dev, generator=gen) * (hi - lo) + lo).half())
        zeros.append(None if case.zero is None else
                     (torch.rand(case.zero.shape, device=dev, generator=gen) * 0.1 - 0.05).half())
    bias = up(case.bias)
    x = up(case.x)
    # outputs: [R][world][M][N] so that with N > 1 the kernel writes its slice of the gather buffer
    fused = world > 1 and args.exchange == "fused"
    window, peers, lay = None, {}, None
    exchange_note = ""
    if fused:
        # the gather buffers live in a window the other ranks map; every rank maps all the others.
        # If any rank cannot (no peer access between two GPUs), all ranks fall back to the all-gather.
        lay = exchange.layout(world, case.M, case.N, buffers=R)
        why = ""
        try:
            window = exchange.Window(lay.total_bytes)
        except Exception as e:  # noqa: BLE001
            why = f"window: {e}"
        handles = [None] * world
        dist.all_gather_object(handles, window.handle if window else None)
        if not why and all(h is not None for h in handles):
            try:
                peers = {r: exchange.PeerWindow(h) for r, h in enumerate(handles) if r != rank}
            except Exception as e:  # noqa: BLE001
                why = f"peer mapping: {e}"
        elif not why:
            why = "a peer has no window"
        flag = torch.tensor([0 if why else 1], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            reasons = [None] * world
            dist.all_gather_object(reasons, why)
            exchange_note = "fused exchange unavailable (" + "; ".join(sorted({r for r in reasons if r})) + "): NCCL all-gather instead"
            for pw in peers.values():
                pw.close()
            peers, fused = {}, False
    if fused:
        outs = None
        out_views = [window.tensor(lay.segment_offset(r, 0), (world, case.M, case.N)) for r in range(R)]
        dist.barrier()
    else:
        outs = torch.zeros(R, world, case.M, case.N, dtype=torch.float16, device=dev)
        out_views = [outs[r] for r in range(R)]
    def build_ops(use_fused, views):
        built, arr = [], 0
        for r in range(R):
            a = api.Arguments(M=case.M, N=case.N, K=case.K, weights=weights[r], x=x, scale=scales[r], zero=zeros[r],
                              bias=bias, out=views[r][rank], weight_bits=case.bits, quant_op=case.quant_op,
                              group_size=case.group_size, variant=variant, flags=0 if args.no_pdl else 8,
                              prefetch=weights[(r + 1) % R] if args.prefetch_next else None)
            if use_fused:
                order = sorted(peers)
                a.peer_out = tuple(peers[q].ptr + lay.segment_offset(r, rank) for q in order)
                a.peer_flag = tuple(peers[q].ptr + exchange.counter_offset(rank) for q in order)
                # the consumer side rides in the next call's kernel: call i+1 reads x only after the
                # peers' slices of call i have landed (equal shards: every rank launches the same grid)
                if r == 0:
                    probe = api.GemvAdaptor()
                    probe.initialize(a)
                    arr = probe.launch_info.grid  # per call and source: one per thread block of that rank's launch
                a.wait_flag = window.ptr + exchange.COUNTERS_OFFSET
                a.wait_state = window.ptr + exchange.STATE_OFFSET
                a.wait_delta = arr
                a.wait_sources = exchange.source_mask(world, rank)
            if not args.no_workspace:
                a.workspace = api.GemvAdaptor.allocate_workspace(a)
            op = api.GemvAdaptor()
            op.initialize(a)
            built.append(op)
        return built, arr

    ops, arrivals = build_ops(fused, out_views)
    info = ops[0].launch_info
    lib = _lib.load()

    def one_step():
        for r in range(R):
            ops[r].run()
            if world > 1 and not fused and args.exchange == "nccl":
                dist.all_gather_into_tensor(outs[r].view(-1), outs[r, rank].reshape(-1))
        if fused:  # the step's last call has no next kernel to wait in: one wait kernel per step
            _lib.check(lib.mgv_wait_arrivals(C.c_void_p(window.ptr + exchange.COUNTERS_OFFSET),
                                             C.c_void_p(window.ptr + exchange.SEEN_OFFSET),
                                             C.c_uint32(exchange.source_mask(world, rank)), C.c_uint32(R * arrivals),
                                             C.c_void_p(int(torch.cuda.current_stream().cuda_stream))))

    one_step()
    torch.cuda.synchronize()
    err = api.device_error_state()
    if world > 1:
        # a bounded wait that gave up on any rank (a peer that never delivered) sends ALL ranks to the all-gather
        t = torch.tensor([err], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err = int(t.item())
    if err != 0 and fused:
        exchange_note = f"fused exchange timed out in the first step (device error word 0x{err:x}): NCCL all-gather instead"
        fused = False
        outs = torch.zeros(R, world, case.M, case.N, dtype=torch.float16, device=dev)
        out_views = [outs[r] for r in range(R)]
        ops, arrivals = build_ops(False, out_views)
        info = ops[0].launch_info
    elif err != 0:
        raise RuntimeError("a device-side wait timed out")

    # ---- correctness of set 0 on a row sample, against the CPU checker ----
    one_step()
    torch.cuda.synchronize()
    if api.device_error_state() != 0:
        raise RuntimeError("a device-side wait timed out")
    from oracle import oracle
    rows = np.arange(0, case.N, max(1, case.N // 256))
    sub_w = case.w_unpacked[rows]
    sub = synth.Case(M=case.M, N=rows.size, K=case.K, bits=case.bits, quant_op=case.quant_op, group_size=case.group_size,
                     w=synth.pack_int4_np(sub_w) if case.bits == 4 else np.ascontiguousarray(sub_w), w_unpacked=sub_w,
                     x=case.x, scale=np.ascontiguousarray(case.scale[:, rows]),
                     zero=None if case.zero is None else np.ascontiguousarray(case.zero[:, rows]), zero_i8=None,
                     bias=None if case.bias is None else case.bias[rows])
    want = oracle.gemv(sub.w, sub.x, sub.scale, bits=sub.bits, group_size=sub.group_size, zero=sub.zero, bias=sub.bias,
                       n_threads=oracle.max_threads())
    ok, max_abs, max_rel = synth.check_close(out_views[0][rank].cpu().numpy()[:, rows], want, sub)
    if not ok:
        raise RuntimeError(f"bench output differs from the CPU checker: max_abs={max_abs} max_rel={max_rel}")
    if world > 1 and args.exchange != "none":
        # the exchange itself: every rank must hold every other rank's slice of set 0, bit for bit
        ref = torch.zeros(world, case.M, case.N, dtype=torch.float16, device=dev)
        dist.all_gather_into_tensor(ref.view(-1), out_views[0][rank].reshape(-1).clone())
        if not torch.equal(ref, out_views[0]):
            raise RuntimeError("the gathered output differs from the ranks' own slices")

    # ---- CUDA graphs: several passes over the R layers per graph, `reps` replays per step ----
    import math
    passes = 1 if args.no_graph else max(1, 288 // R)

    def capture(fn, n_passes):
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(n_passes):
                fn()
        return g

    graph = None if args.no_graph else capture(one_step, passes)
    replay = graph.replay if graph is not None else one_step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(n):
            fn()
        a1.record()
        torch.cuda.synchronize()
        return a0.elapsed_time(a1)

    for _ in range(3):
        replay()
    barrier()
    est = torch.tensor([timed(replay, 4) / 4], device=dev)          # ms per replay
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    reps = max(1, int(math.ceil(50.0 / max(float(est.item()), 1e-4))))  # a step lasts at least 50 ms

    def step():
        for _ in range(reps):
            replay()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    marks[0].record()
    for i in range(args.steps):
        step()
        marks[i + 1].record()
    barrier()
    ms = marks[0].elapsed_time(marks[-1])
    step_ms = [marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps)]
    clocks = None
    if rank == 0:
        t_end = time.perf_counter() + 3.0   # a very short run: keep the load up until a few samples exist
        while world == 1 and len(sampler.rows) < 8 and time.perf_counter() < t_end:
            step()
            torch.cuda.synchronize()
        clocks = sampler.stop()
        clocks["note"] = "sampled every 100 ms during the timed region"
    if world > 1:
        tt = torch.tensor([ms, statistics.median(step_ms)], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, med_ms = float(tt[0].item()), float(tt[1].item())
    else:
        med_ms = statistics.median(step_ms)
    calls_per_step = reps * passes * R
    calls = args.steps * calls_per_step
    us_per_call = 1e3 * ms / calls
    value = world * nbytes * calls / (ms * 1e-3) / 1e9
    per_gpu = value / world
    peak, peak_src = peaks()

    # ---- the same chain with every kernel starting only after its predecessor has finished ----
    isolated_us = None
    if world == 1 and not args.no_pdl and not args.no_graph:
        saved = ops
        ops = [api.GemvAdaptor() for _ in range(R)]
        for r in range(R):
            a = saved[r]._keep
            a.flags &= ~8
            ops[r].initialize(a)
            a.flags |= 8
        g_iso = capture(one_step, passes)
        for _ in range(3):
            g_iso.replay()
        n_iso = max(1, reps // 2)
        isolated_us = 1e3 * timed(g_iso.replay, n_iso) / (n_iso * passes * R)
        ops = saved

    # ---- e2e through the host-buffer C ABI ----
    e2e = None
    if not args.no_e2e and world > 1:
        e2e = None  # (set below: the host-buffer call serves one unsharded layer per GPU, not the sharded layer)
    if not args.no_e2e and world == 1:
        layers = []
        n_layers = min(R, 16)
        for r in range(n_layers):
            c = case if r == 0 else synth.config(args.workload, M=args.M, seed=1000 + rank * 100 + r)
            layers.append(api.Linear(c, max_M=case.M))
        xh = torch.from_numpy(case.x.copy()).pin_memory()
        oh = torch.zeros(case.M, case.N, dtype=torch.float16).pin_memory()
        for _ in range(2):
            for l in layers:
                l.forward_host(xh, oh, M=case.M, variant=variant)
        barrier()
        t0 = time.perf_counter()
        n_e2e = 0
        while n_e2e < 2000 and (n_e2e < 200 or time.perf_counter() - t0 < 0.5):
            for l in layers:
                l.forward_host(xh, oh, M=case.M, variant=variant)
                n_e2e += 1
        dt = time.perf_counter() - t0
        calls_per_step_e2e = n_layers
        e2e = {"value": world * nbytes * n_e2e / dt / 1e9, "unit": "GB/s", "us_per_call": 1e6 * dt / n_e2e,
               "h2d_bytes_per_step": calls_per_step_e2e * case.M * case.K * 2,
               "d2h_bytes_per_step": calls_per_step_e2e * case.M * case.N * 2,
               "calls_per_step": calls_per_step_e2e,
               "note": "mgv_linear_forward_host per call: x read from the pinned host buffer by a one-block kernel (H2D over PCIe), GEMV as its dependent launch writing the result into the pinned host buffer (D2H over PCIe by the epilogue), wait; one graph launch per call; weights resident"}
        for l in layers:
            l.close()

    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        dt, kind, threads = cpu_gemv_timing(case)
        cpu = {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": kind, "seconds_per_call": dt,
               "sample": "one full call of the workload shape, rows split over all host threads"}
        # the reference's host GEMV as written has no threading: one thread, one full call (bounded: skipped when
        # the all-threads figure says it would take more than about half a minute)
        if dt * threads < 30.0:
            dt1, kind1, _ = cpu_gemv_timing(case, threads=1)
            cpu["as_written_1_thread"] = {"value": nbytes / dt1 / 1e9, "unit": "GB/s", "cores": 1, "kind": kind1,
                                          "seconds_per_call": dt1}

    # ---- the reference's own CUDA kernel, recompiled for this GPU, on the same buffers (N = 1, where it instantiates) ----
    ref_gpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        from oracle import oracle as _oracle
        if (_oracle.have_ref_cuda() and case.bits == 4 and case.M == 1 and case.group_size in (64, 128) and case.bias is None
                and int(case.quant_op) in (2, 3)):
            ref_outs = torch.zeros(R, case.N, dtype=torch.float16, device=dev)

            def ref_step():
                st = int(torch.cuda.current_stream().cuda_stream)
                for r in range(R):
                    _oracle.ref_device_gemv(int(case.quant_op), weights[r].data_ptr(), x.data_ptr(), scales[r].data_ptr(),
                                            zeros[r].data_ptr() if zeros[r] is not None else 0, ref_outs[r].data_ptr(),
                                            case.N, case.K, case.group_size, st)
            ref_step()
            torch.cuda.synchronize()
            agree = bool(synth.check_close(ref_outs[0].cpu().numpy()[None, rows], want, sub)[0])
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                ref_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            rg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(rg):
                ref_step()
            for _ in range(3):
                rg.replay()
            torch.cuda.synchronize()
            n_ref = max(3, min(200, int(20000.0 / max(1.0, R * 45.0))))   # about 20 ms of replays
            ref_us = 1e3 * timed(rg.replay, n_ref) / (n_ref * R)
            ref_gpu = {"us_per_call": ref_us, "value": nbytes / (ref_us * 1e-6) / 1e9, "unit": "GB/s",
                       "matches_cpu_checker": agree,
                       "what": "the reference's GemvAdaptor kernel (SIMT, 64x1x64 tiles, one stage: its test driver's "
                               "configuration) recompiled for sm_100a against CUTLASS 4.5.0, same buffers, same graph replay"}

    _KEEP.extend([graph, ops, window, peers, outs, weights, scales, zeros])
    if rank != 0:
        return None

    # ---- the preprocessing kernel on this layer's weights (2 x bytes: read + write) ----
    prep = None
    if world == 1 and not args.no_cpu_baseline:
        prep = {}
        for name, layout in (("column_major", LayoutType.kColumnMajor), ("row_major", LayoutType.kRowMajor)):
            if layout == LayoutType.kRowMajor and ((case.N * case.bits // 8) % 32 or (case.K * case.bits // 8) % 32):
                continue
            dst = torch.empty_like(raw0)
            run = lambda: api.MixedGemvWeightPreprocessor.run(dst, raw0, (case.K, case.N), layout, qt)
            run()
            torch.cuda.synchronize()
            n_prep = 20  # replayed from a graph: the host side of a call costs more than the kernel on a small layer
            g_prep = capture(run, n_prep)
            g_prep.replay()
            us = 1e3 * timed(g_prep.replay, 5) / (5 * n_prep)
            prep[name] = {"us_per_call": us, "value": 2 * raw0.numel() / (us * 1e-6) / 1e9, "unit": "GB/s",
                          "frac_of_peak": 2 * raw0.numel() / (us * 1e-6) / 1e9 / peak}
        prep["note"] = ("mgv_preprocess_weights on one layer of the workload; algorithmic bytes = 2 x weight bytes; the source "
                        "of consecutive calls is the same buffer, which fits L2 for small layers")

    traffic, traffic_kernel = traffic_bytes(case)
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms / args.steps, "ms_per_step_median": med_ms, "us_per_call": us_per_call,
        "isolated_us_per_call": isolated_us, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 x int%d -> f32 accumulate" % case.bits, "data": "synthetic",
        "config": {"workload": workload_string(case),
                   **({"sharding": f"N-split layer of N={case.N * world}, output slices exchanged by "
                                   + ("the kernels themselves (epilogue stores into the peers' gather buffers over NVLink and counts its blocks in; the next call's kernel waits, bounded, for the peers' counts before it reads x)"
                                      if fused else "nothing (kernels only, no exchange)" if args.exchange == "none"
                                      else "an NCCL all-gather after every call")} if world > 1 else {}),
                   "calls_per_step": calls_per_step, "layers": R, "passes_per_graph": passes, "graph_replays_per_step": reps,
                   "l2_policy": f"{R} distinct resident layers = {R * nbytes / 2**20:.0f} MiB "
                                f"(L2 is {l2 / 2**20:.0f} MiB): inputs larger than L2",
                   "variant": Variant(info.variant).name, "grid": info.grid, "block": info.block, "stages": info.stages,
                   "smem_bytes": info.smem_bytes, "split_tiles": info.split_tiles, "cuda_graph": graph is not None,
                   "programmatic_dependent_launch": not args.no_pdl, "prefetch_hint": bool(args.prefetch_next),
                   **({"exchange_note": exchange_note} if exchange_note else {}),
                   "check": {"rows": int(rows.size), "max_abs": max_abs, "max_rel": max_rel}},
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "traffic": traffic,
                     "traffic_source": (f"recorded from an ncu capture of one launch of {traffic_kernel} on this workload "
                                        "(dram__bytes_read.sum + dram__bytes_write.sum); not measured by this run") if traffic else None,
                     "peak_source": peak_src, "bytes_per_launch": nbytes,
                     "note": "per GPU; achieved = algorithmic bytes per launch / average launch-to-launch time over the timed region"},
        "e2e": e2e,
        **({"e2e_note": "null at N > 1: the host-buffer entry point serves one unsharded layer per GPU, which would time N "
                        "independent replicas, not the sharded layer"} if world > 1 else {}),
        "cpu_baseline": cpu, "reference_gpu": ref_gpu, "preprocess": prep,
        "gpu_launches": calls + (args.steps * reps * passes if fused else 0), "clocks": clocks,
    }
    return line


def sharded_layers(args, world):
    """N > 1: the two 70B-class layers of the benchmark configs, each cut over all N GPUs (strong
    scaling): gate/up (K = 8192, N = 57344) over N, down (K = 28672, N = 8192) over K.  Per layer:
    the kernels alone (no exchange), the fused exchange and the NCCL collective."""
    out = {}
    for name, split, workload, dims in (("c5_gateup_n_split", "n", "c5_gateup", dict(N=57344 // world)),
                                        ("c5_down_k_split", "k", "c5_down", dict(K=28672 // world))):
        entry = {}
        for exch in ("none", "fused", "nccl"):
            sub = argparse.Namespace(**vars(args))
            sub.workload, sub.split, sub.exchange = workload, split, exch
            sub.N, sub.K = dims.get("N", 0), dims.get("K", 0)
            sub.steps, sub.warmup, sub.no_e2e, sub.no_cpu_baseline, sub.sets, sub.M = 3, 3, True, True, 0, 1
            line = run_ours_ksplit(sub) if split == "k" else run_ours(sub)
            if line is not None:
                entry[{"none": "kernels_only", "fused": "fused_exchange", "nccl": "nccl_exchange"}[exch]] = {
                    "us_per_call": line["us_per_call"], "aggregate_gbs": line["value"], "per_gpu_frac_of_peak": line["roofline"]["frac"],
                    "workload": line["config"]["workload"], "sharding": line["config"].get("sharding"),
                    "check": line["config"].get("check")}
        out[name] = entry
    return out


if __name__ == "__main__":
    a = parse()
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    if a.impl == "reference":
        run_reference(a)
    else:
        k_split = a.split == "k" and world_size > 1
        line = run_ours_ksplit(a) if k_split else run_ours(a)
        if world_size > 1 and not a.no_extra and not k_split and a.workload == DEFAULT_WORKLOAD and not a.N and not a.K:
            extra = sharded_layers(a, world_size)
            if line is not None:
                line["sharded_layers"] = extra
        if line is not None:
            print(json.dumps(line))
        finish()
