"""RMSNorm: x / sqrt(mean(x^2) + eps) * weight, statistics in float32
(the reference's `rms_norm`, src/model.rs:200-214; src/cuda/kernels/rmsnorm.cu:32-38).

The part owns the fusion with the residual addition: the stream's pending sub-layer
output is added to the float32 residual in the same pass that normalises it
(the reference runs `add.cu`, `rmsnorm.cu` and `f32_to_f16.cu` one after the other,
src/cuda/model.rs:685-790).
"""
from __future__ import annotations

import torch

from .base import Norm, register_norm
from .spec import NormSpec, ParamDecl


class RMSNorm(Norm):
    @staticmethod
    def params(spec: NormSpec):
        return {"weight": ParamDecl((spec.size,), "norm")}

    def __init__(self, spec: NormSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        # Norm weights are tiny; float32 keeps a 32-bit file exact and widens a
        # bfloat16 file without loss.
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def add_norm(self, resid, delta, ctx, rows=None):
        n = resid.shape[0] if rows is None else rows.shape[0]
        out = self.ops.new_rows(n, self.spec.size, self.dtype, resid.device)
        self.ops.add_rmsnorm(resid, delta, self.weight, self.spec.eps, out, rows)
        return out


    def norm(self, x, ctx):
        out = self.ops.new_rows(x.shape[0], self.spec.size, self.dtype, x.device)
        self.ops.add_rmsnorm(None, x, self.weight, self.spec.eps, out, None)
        return out


register_norm("rmsnorm", RMSNorm)
