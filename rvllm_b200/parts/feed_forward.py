"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)) (the reference's `swiglu_ffn`,
src/model.rs:320-335).

gate and up are stored as one [2F, hidden] matrix so that they are one matrix
product; the activation kernel reads both halves of its output row.  (The reference
runs two products and `silu_gate_multiply.cu`, src/cuda/model.rs:740-760.)
"""
from __future__ import annotations

import torch

from .base import FeedForward, register_feed_forward
from .spec import ParamDecl, SwiGLUSpec


class SwiGLU(FeedForward):
    @staticmethod
    def params(spec: SwiGLUSpec):
        n = spec.names
        return {
            n.get("gate", "gate.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
            n.get("up", "up.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
            n.get("down", "down.weight"): ParamDecl((spec.hidden, spec.ffn_dim), "linear"),
        }

    def __init__(self, spec: SwiGLUSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = spec.names
        gate = tensors[n.get("gate", "gate.weight")]
        up = tensors[n.get("up", "up.weight")]
        self.gate_up = torch.cat([gate, up.to(gate.dtype)], dim=0).contiguous()
        self.down = tensors[n.get("down", "down.weight")].contiguous()

    def forward(self, normed, ctx):
        gate_up = self.ops.linear(normed, self.gate_up, out_dtype=self.dtype)
        act = self.ops.new_rows(normed.shape[0], self.spec.ffn_dim, self.dtype, normed.device)
        self.ops.swiglu(gate_up, act)
        return self.ops.linear(act, self.down, out_dtype=self.dtype)


register_feed_forward("swiglu", SwiGLU)
