"""CPU tests of the multi-GPU host logic: shard planning, the layout facts the N split relies on,
and the two exchange patterns run by world_size-2 gloo ranks with the CPU checker standing in for
the local kernel."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from mixed_gemv_b200 import sharded, synth
from mixed_gemv_b200.enums import WeightOnlyQuantOp as Q


def test_column_plan_covers_n_on_aligned_boundaries():
    for N, world in ((57344, 8), (57344, 2), (11008, 4), (4096, 8), (192, 3)):
        shards = [sharded.plan_column_split(N, world, r) for r in range(world)]
        assert shards[0].begin == 0 and shards[-1].end == N
        for a, b in zip(shards, shards[1:]):
            assert a.end == b.begin
        assert all(s.begin % 64 == 0 and s.size > 0 for s in shards)
        assert max(s.size for s in shards) - min(s.size for s in shards) <= 64
    assert [sharded.plan_column_split(57344, 8, r).size for r in range(8)] == [7168] * 8


def test_row_plan_respects_groups():
    for K, world, g in ((28672, 8, 128), (28672, 2, 128), (8192, 4, 64), (11008, 2, 128)):
        shards = [sharded.plan_row_split(K, world, r, g) for r in range(world)]
        assert shards[0].begin == 0 and shards[-1].end == K
        assert all(s.begin % max(g, 64) == 0 for s in shards)
    assert [sharded.plan_row_split(28672, 8, r, 128).size for r in range(8)] == [3584] * 8


def test_plans_refuse_bad_requests():
    with pytest.raises(sharded.ShardError):
        sharded.plan_column_split(100, 2, 0)          # N not a multiple of 64
    with pytest.raises(sharded.ShardError):
        sharded.plan_column_split(64, 2, 0)           # fewer blocks than ranks
    with pytest.raises(sharded.ShardError):
        sharded.plan_column_split(128, 2, 2)          # rank out of range
    with pytest.raises(sharded.ShardError):
        sharded.plan_row_split(4096 + 64, 2, 0, 128)  # K not on a group boundary
    with pytest.raises(sharded.ShardError):
        sharded.plan_row_split(128, 4, 0, 128)


def test_column_shard_is_a_contiguous_byte_range_of_the_preprocessed_buffer():
    c = synth.make_case(1, 256, 512, bits=4, quant_op=Q.FINEGRAINED_SCALE_ONLY, group_size=128, seed=2)
    full = oracle.preprocess_weights(c.w, (c.K, c.N), oracle.COLUMN_MAJOR, oracle.W4_A16)
    for world in (2, 4):
        for r in range(world):
            sh = sharded.plan_column_split(c.N, world, r)
            local = sharded.slice_case_columns(c, sh)
            lo, hi = sharded.column_shard_bytes(sh, c.K, 4)
            pre = oracle.preprocess_weights(local.w, (local.K, local.N), oracle.COLUMN_MAJOR, oracle.W4_A16)
            assert np.array_equal(pre, full[lo:hi])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, mode, fail_rank, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = synth.make_case(2, 256, 1024, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=128, zeros="f16",
                            bias=True, x_dist="normal", seed=7)
        if mode == "column":
            sh = sharded.plan_column_split(c.N, world, rank)
            if rank == fail_rank:   # a rank whose shard does not match its weights must fail on the host
                sh = sharded.Shard(rank, world, sh.begin, sh.end - 64)
            local = sharded.slice_case_columns(c, sharded.plan_column_split(c.N, world, rank))
            if sh.size != local.N:
                raise sharded.ShardError("shard size mismatch")
            y = oracle.gemv(local.w, local.x, local.scale, bits=4, group_size=128, zero=local.zero, bias=local.bias)
            gathered = torch.zeros(world, c.M, local.N, dtype=torch.float16)
            dist.all_gather_into_tensor(gathered.view(-1), torch.from_numpy(y).reshape(-1))
            got = np.concatenate([gathered[r].numpy() for r in range(world)], axis=1)
        else:
            sh = sharded.plan_row_split(c.K, world, rank, c.group_size)
            local = sharded.slice_case_rows(c, sh)
            _, part = oracle.gemv(local.w, local.x, local.scale, bits=4, group_size=128, zero=local.zero, bias=None,
                                  want_f32=True)
            t = torch.from_numpy(part.copy())
            dist.all_reduce(t)
            got = (t.numpy() + c.bias.astype(np.float32)[None, :]).astype(np.float16)
        want = oracle.gemv(c.w, c.x, c.scale, bits=4, group_size=128, zero=c.zero, bias=c.bias)
        if mode == "column":
            assert np.array_equal(got.view(np.uint16), want.view(np.uint16))       # rows are independent: bit-exact
        else:
            assert synth.check_close(got, want, c)[0]                              # fp32 sum order differs
            assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 4 * np.spacing(np.float16(np.abs(want).max()))
        open(os.path.join(out_dir, f"ok_{mode}_{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["column", "row"])
def test_two_gloo_ranks_reproduce_the_unsharded_result(tmp_path, mode):
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, mode, -1, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok_{mode}_0", f"ok_{mode}_1"]


def test_a_rank_with_a_wrong_shard_fails_on_the_host(tmp_path):
    """Failure is injected on the host: rank 1 raises before any collective; the parent sees the error."""
    port = _free_port()
    with pytest.raises(Exception):
        mp.spawn(_rank_main, args=(2, port, "column", 1, str(tmp_path)), nprocs=2, join=True)
    assert not os.path.exists(os.path.join(tmp_path, "ok_column_1"))
