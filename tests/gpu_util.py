"""Helpers shared by the GPU parity tests: run one seeded case through the C ABI."""
import numpy as np
import torch

from oracle import oracle
from mixed_gemv_b200 import api
from mixed_gemv_b200.enums import LayoutType, QuantType, Variant, WeightOnlyQuantOp as Q


class DeviceCase:
    """A synth.Case uploaded and preprocessed on the GPU."""

    def __init__(self, case):
        self.case = c = case
        raw = torch.from_numpy(np.ascontiguousarray(c.w).view(np.uint8).ravel().copy()).cuda()
        self.w = torch.empty_like(raw)
        api.MixedGemvWeightPreprocessor.run(self.w, raw, (c.K, c.N), LayoutType.kColumnMajor,
                                            QuantType.W4_A16 if c.bits == 4 else QuantType.W8_A16)
        self.x = torch.from_numpy(c.x.copy()).cuda()
        self.scale = torch.from_numpy(c.scale.copy()).cuda()
        self.zero = None if c.zero is None else torch.from_numpy(c.zero.copy()).cuda()
        self.bias = None if c.bias is None else torch.from_numpy(c.bias.copy()).cuda()

    def arguments(self, M=None, variant=Variant.AUTO, out=None, flags=0, alpha=1.0, beta=1.0,
                  workspace="auto", hints=0):
        c = self.case
        M = c.M if M is None else M
        if out is None:
            dt = torch.float32 if flags & 1 else torch.float16
            out = torch.full((M, c.N), float("nan"), dtype=dt, device="cuda")
        a = api.Arguments(M=M, N=c.N, K=c.K, weights=self.w, x=self.x, scale=self.scale, out=out,
                          zero=self.zero, bias=self.bias, weight_bits=c.bits, quant_op=c.quant_op,
                          group_size=c.group_size, variant=variant, flags=flags, alpha=alpha, beta=beta, hints=hints)
        if workspace == "auto":
            a.workspace = api.GemvAdaptor.allocate_workspace(a)
        elif workspace is not None:
            a.workspace = workspace
        return a

    def run(self, **kw) -> np.ndarray:
        a = self.arguments(**kw)
        api.GemvAdaptor()(a)
        torch.cuda.synchronize()
        assert api.device_error_state() == 0
        return a.out.cpu().numpy()


def oracle_out(case, M=None, alpha=1.0, beta=1.0, want_f32=False, threads=None):
    c = case
    M = c.M if M is None else M
    return oracle.gemv(c.w, c.x[:M], c.scale, bits=c.bits, group_size=c.group_size, zero=c.zero,
                       bias=c.bias, alpha=alpha, beta=beta, want_f32=want_f32,
                       n_threads=threads or oracle.max_threads())
