"""The reference's own CUDA kernel (its GemvAdaptor in its test driver's configuration, recompiled
for sm_100a into oracle/_ref/libmgv_ref_cuda.so) run on the same device buffers as the library:
it must agree with the host checker, and the library's SIMT family -- which rounds where the
reference rounds -- must agree with it to within the order of the fp32 additions."""
import numpy as np
import pytest
import torch

from mixed_gemv_b200 import synth
from mixed_gemv_b200.enums import Variant, WeightOnlyQuantOp as Q
from oracle import oracle
from tests.gpu_util import DeviceCase, oracle_out

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("op,group,N,K", [(Q.FINEGRAINED_SCALE_ONLY, 128, 1024, 2048), (Q.FINEGRAINED_SCALE_AND_ZEROS, 64, 1088, 4096),
                                          (Q.FINEGRAINED_SCALE_ONLY, 128, 11008, 4096)])
def test_reference_kernel_and_library_agree(cuda_lib, op, group, N, K):
    if not oracle.have_ref_cuda():
        pytest.skip("oracle/_ref/libmgv_ref_cuda.so was not built")
    c = synth.make_case(1, N, K, bits=4, quant_op=op, group_size=group, zeros="f16", bias=False, x_dist="uniform", seed=N % 71)
    d = DeviceCase(c)
    ref_out = torch.zeros(1, N, dtype=torch.float16, device="cuda")
    oracle.ref_device_gemv(int(op), d.w.data_ptr(), d.x.data_ptr(), d.scale.data_ptr(),
                           d.zero.data_ptr() if d.zero is not None else 0, ref_out.data_ptr(), N, K, group,
                           int(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    ref_np = ref_out.cpu().numpy()
    want = oracle_out(c)
    ok, max_abs, max_rel = synth.check_close(ref_np, want, c)
    assert ok, ("reference kernel vs host checker", max_abs, max_rel)
    top = float(np.abs(want.astype(np.float32)).max())
    for variant, bound in ((Variant.SIMT, 2 * float(np.spacing(np.float16(top))) + 1e-6 * top), (Variant.MMA, 5e-4 * top + 2 * float(np.spacing(np.float16(top))))):
        got = d.run(variant=variant)
        assert synth.check_close(got, want, c)[0]
        diff = float(np.abs(got.astype(np.float32) - ref_np.astype(np.float32)).max())
        assert diff <= bound, (variant, diff, bound)
