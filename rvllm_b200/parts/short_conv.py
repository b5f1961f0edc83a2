"""Gated short convolution, the LFM2 mixer of the non-attention layers.

In the reference's order (src/model.rs:659-688): bcx = in_proj(normed), three chunks
B, C, x in this order; bx = B * x; each request's window is its taps-1 previous bx
rows (zeros before position 0, src/conv_cache.rs:69-71) followed by the new rows;
conv[t, c] = sum_k filter[c, k] * window[t + k, c], tap taps-1 on the token itself
(src/cuda/kernels/short_conv.cu:39-42); y = C * conv; out = out_proj(y); the new
state is the window's last taps-1 rows (src/conv_cache.rs:103-105).

With `bias` (an option the reference lacks) in_proj, the convolution and out_proj
each add their bias where a linear layer or a convolution does.

The state is one float32 record [taps-1, hidden] per request in a slot of the cache
manager, where the reference keeps hash maps of small tensors keyed by (sequence,
layer) (src/conv_cache.rs:33-41).  Gate, taps, state load and state store are one
kernel for any mixture of prompt portions and single tokens.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed, register_mixer
from .spec import ParamDecl, ShortConvSpec


class ShortConv(Mixer):
    @staticmethod
    def _names(spec):
        n = spec.names
        return {k: n.get(k, k) for k in
                ("in_proj.weight", "conv.weight", "out_proj.weight",
                 "in_proj.bias", "conv.bias", "out_proj.bias")}

    @staticmethod
    def params(spec: ShortConvSpec, owns_cache: bool = True):
        n = ShortConv._names(spec)
        h, k = spec.hidden, spec.taps
        p = {n["in_proj.weight"]: ParamDecl((3 * h, h), "linear"),
             n["conv.weight"]: ParamDecl((h, k), "conv", alt_shapes=((h, 1, k),)),
             n["out_proj.weight"]: ParamDecl((h, h), "linear")}
        if spec.bias:
            p[n["in_proj.bias"]] = ParamDecl((3 * h,), "bias")
            p[n["conv.bias"]] = ParamDecl((h,), "bias")
            p[n["out_proj.bias"]] = ParamDecl((h,), "bias")
        return p

    @staticmethod
    def cache_need(spec: ShortConvSpec):
        if spec.taps <= 1:
            return None
        return StateNeed((spec.taps - 1, spec.hidden))

    def __init__(self, spec: ShortConvSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        f32 = torch.float32
        self.w_in = tensors[n["in_proj.weight"]].contiguous()
        self.w_out = tensors[n["out_proj.weight"]].contiguous()
        self.filter = tensors[n["conv.weight"]].to(f32).reshape(spec.hidden, spec.taps).contiguous()
        self.b_in = self.b_conv = self.b_out = None
        if spec.bias:
            self.b_in = tensors[n["in_proj.bias"]].to(f32).contiguous()
            self.b_conv = tensors[n["conv.bias"]].to(f32).contiguous()
            self.b_out = tensors[n["out_proj.bias"]].to(f32).contiguous()

    def forward(self, normed, ctx, cache):
        if cache is not None and not cache.owns:
            raise ValueError("short_conv: a convolution state cannot be shared between calls")
        proj = self.ops.linear(normed, self.w_in, out_dtype=self.dtype)
        y = self.ops.new_rows(normed.shape[0], self.spec.hidden, self.dtype, normed.device)
        self.ops.short_conv(proj, self.filter, self.b_in, self.b_conv,
                            cache.state if cache is not None else None, ctx, y)
        out = self.ops.linear(y, self.w_out, out_dtype=self.dtype)
        if self.b_out is not None:
            self.ops.add_bias(out, self.b_out)
        return out


register_mixer("short_conv", ShortConv)
