"""The allocation-free entry point, mgv_gemv_static_scratch, against mgv_gemv.

Some callers cannot give the library scratch memory because they cannot allocate at all at the
moment they call: a stream capture is in progress, or a plug-in hook runs under a fixed memory
budget.  For them the split-K scratch is an array inside the library image.  This file is named so
that pytest collects it last: the array is shared by every call in the process, so the test must
hold both in a fresh process and after everything else has run.
"""
import numpy as np
import pytest
import torch

from mixed_gemv_b200 import _lib as L, api, synth
from mixed_gemv_b200.enums import Status, Variant, WeightOnlyQuantOp as Q
from mixed_gemv_b200._lib import MgvError
from tests.gpu_util import DeviceCase, oracle_out

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", [Variant.MMA, Variant.SIMT], ids=["mma", "simt"])
def test_static_scratch_matches_caller_owned_scratch_twice_in_a_row(cuda_lib, variant):
    # HINT_DEAL_ITEMS makes the library cut row tiles between thread blocks, so that the scratch is really used
    c = synth.make_case(2, 256, 11008, bits=4, quant_op=Q.FINEGRAINED_SCALE_AND_ZEROS, group_size=128, zeros="f16",
                        bias=True, x_dist="normal", seed=17)
    d = DeviceCase(c)
    a = d.arguments(variant=variant, hints=L.HINT_DEAL_ITEMS)   # caller-owned scratch, the existing entry point
    assert a.workspace is not None
    op = api.GemvAdaptor()
    op.initialize(a)
    assert op.launch_info.split_tiles > 0
    op.run()
    torch.cuda.synchronize()
    want = a.out.cpu().numpy().copy()
    assert np.isfinite(want.astype(np.float32)).all()
    checker = oracle_out(c)                           # ... and the existing entry point against the CPU checker
    assert synth.check_close(want, checker, c)[0]

    b = d.arguments(variant=variant, workspace=None, hints=L.HINT_DEAL_ITEMS)  # no scratch from the caller at all
    op2 = api.GemvAdaptor()
    op2.initialize(b)
    for attempt in range(2):                          # two calls in a row share the built-in array
        b.out.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]    # the driver's view: any cudaMalloc would lower it
        op2.run_static_scratch()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        got = b.out.cpu().numpy()
        # same kernel, same dealing, same fixed summation order: the two entry points agree bit for bit,
        # which is inside the tolerance the other GPU tests use (synth.check_close)
        assert synth.check_close(got, want, c)[0], attempt
        assert synth.check_close(got, checker, c)[0], attempt
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), attempt
    assert api.device_error_state() == 0


def test_static_scratch_refuses_shapes_beyond_its_array(cuda_lib):
    # Sizing needs no real buffers of that size: only N enters the scratch requirement, and N is
    # chosen so that the per-tile arrival counters ALONE (4 bytes per 32 rows) exceed the 4 MiB
    # array on any device.  The size query launches nothing; the call below is made only once the
    # query has confirmed that the refusal must fire, so no kernel can ever run on the placeholders.
    N, K = 32 * 1_100_000, 512
    t = torch.zeros(16, dtype=torch.float16, device="cuda")
    a = api.Arguments(M=1, N=N, K=K, weights=t.view(torch.uint8), x=t, scale=t, out=t, weight_bits=4,
                      quant_op=Q.PER_COLUMN_SCALE_ONLY, group_size=K, hints=L.HINT_DEAL_ITEMS)
    need = api.GemvAdaptor.get_workspace_size(a)
    if need <= (4 << 20):
        pytest.skip(f"the planner asks for {need} bytes only: nothing to refuse")
    op = api.GemvAdaptor()
    op._args = api.GemvAdaptor._to_c(a)               # skip initialize(): the buffers are placeholders
    with pytest.raises(MgvError) as e:
        op.run_static_scratch()
    assert e.value.status == Status.WORKSPACE_TOO_SMALL
    assert "built-in array" in str(e.value)
