"""Two-GPU test of the sharded layers (NCCL): N split + all-gather and K split + all-reduce against
the unsharded CPU checker.  Skipped on boxes with one GPU; the same logic runs on CPU with gloo in
tests/test_sharded_cpu.py."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, out_dir):
    import torch.distributed as dist
    from oracle import oracle
    from mixed_gemv_b200 import sharded, synth
    from mixed_gemv_b200.enums import WeightOnlyQuantOp as Q
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        c = synth.make_case(2, 1024, 2048, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=128, zeros="f16",
                            bias=True, x_dist="normal", seed=3)
        want = oracle.gemv(c.w, c.x, c.scale, bits=4, group_size=128, zero=c.zero, bias=c.bias, n_threads=4)
        # N split
        sh = sharded.plan_column_split(c.N, world, rank)
        layer = sharded.ColumnParallelGemv(sharded.slice_case_columns(c, sh), c.N, sh, max_M=2)
        x = torch.from_numpy(c.x.copy()).cuda()
        g = layer.forward(x, M=2)
        torch.cuda.synchronize()
        got = np.concatenate([g[r].cpu().numpy() for r in range(world)], axis=1)
        assert synth.check_close(got, want, c)[0]
        # the same layer built from tensors that already live on the device (a caller's own resident shard)
        ds = sharded.DeviceShard.from_tensors(layer.w, layer.scale, N=sh.size, K=c.K, bits=4, quant_op=c.quant_op,
                                              group_size=c.group_size, zero=layer.zero, bias=layer.bias)
        layer2 = sharded.ColumnParallelGemv(ds, c.N, sh, max_M=2)
        g2 = layer2.forward(x, M=2)
        torch.cuda.synchronize()
        assert torch.equal(g2, g)
        # K split
        sk = sharded.plan_row_split(c.K, world, rank, c.group_size)
        local = sharded.slice_case_rows(c, sk)
        rl = sharded.RowParallelGemv(local, sk, max_M=2)
        out = rl.forward(torch.from_numpy(local.x.copy()).cuda(), M=2)
        torch.cuda.synchronize()
        assert synth.check_close(out.cpu().numpy(), want, c)[0]
        # N split with the exchange fused into the kernel (peer stores + arrival counters, no collective)
        fl = sharded.FusedColumnParallelGemv(sharded.slice_case_columns(c, sh), c.N, sh, max_M=2)
        for call in range(5):  # both gather buffers, several rounds of the counters
            # (inputs of every call differ, but stay of order one: the stated absolute tolerance assumes that)
            xs = torch.from_numpy((c.x * (1 + call / 8)).astype(np.float16)).cuda()
            g = fl.forward(xs, M=2)
            torch.cuda.synchronize()
            got = np.concatenate([g[r].cpu().numpy() for r in range(world)], axis=1)
            want_c = oracle.gemv(c.w, (c.x * (1 + call / 8)).astype(np.float16), c.scale, bits=4, group_size=128,
                                 zero=c.zero, bias=c.bias, n_threads=4)
            assert synth.check_close(got, want_c, c)[0], f"fused exchange, call {call}"
        from mixed_gemv_b200 import api
        assert api.device_error_state() == 0
        fl.close()
        # the same with the wait riding in the next call's kernel (no kernel between the calls)
        fc = sharded.FusedColumnParallelGemv(sharded.slice_case_columns(c, sh), c.N, sh, max_M=2, chained=True)
        xs = [torch.from_numpy((c.x * (1 + k / 8)).astype(np.float16)).cuda() for k in range(6)]
        bufs = [fc.forward(xs[k], M=2, complete=(k % 3 == 2)) for k in range(6)]   # waits after calls 2 and 5
        torch.cuda.synchronize()
        for k in (4, 5):   # the two buffers hold the last two calls
            got = np.concatenate([bufs[k][r].cpu().numpy() for r in range(world)], axis=1)
            want_c = oracle.gemv(c.w, (c.x * (1 + k / 8)).astype(np.float16), c.scale, bits=4, group_size=128,
                                 zero=c.zero, bias=c.bias, n_threads=4)
            assert synth.check_close(got, want_c, c)[0], f"chained exchange, call {k}"
        assert api.device_error_state() == 0
        fc.close()
        # K split with the partials exchanged by the kernels and added in rank order on every rank
        fr = sharded.FusedRowParallelGemv(local, sk, max_M=2)
        xl = torch.from_numpy(local.x.copy()).cuda()
        for call in range(3):
            out = fr.forward(xl, M=2)
            torch.cuda.synchronize()
            assert synth.check_close(out.cpu().numpy(), want, c)[0], f"fused K split, call {call}"
        mine = out.clone()
        both = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        assert all(torch.equal(b, mine) for b in both)     # same order of addition everywhere: same bits
        assert api.device_error_state() == 0
        fr.close()
        open(os.path.join(out_dir, f"ok_{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gpus_column_and_row_split(cuda_lib, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_rank_main, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok_0", "ok_1"]
