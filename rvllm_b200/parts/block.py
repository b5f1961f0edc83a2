"""Arrangements: how a block wires its norms, mixer and feed-forward.

"pre_norm": h = x + mixer(norm(x)); out = h + ffn(norm(h)) (the reference's
`Layer::forward`, src/model.rs:556-585, without the post-norms that LFM2 does not
use).  The residual stream is float32; each sub-layer's output stays pending and is
added by the next norm's kernel.
"""
from __future__ import annotations

from .base import (Arrangement, Stream, feed_forward_class, mixer_class, norm_class,
                   register_arrangement)
from .spec import BlockSpec


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class PreNormBlock(Arrangement):
    @staticmethod
    def params(spec: BlockSpec, owns_cache: bool = True):
        """Full tensor names -> declarations for one block."""
        out = {}
        mixer = mixer_class(spec.mixer.kind)
        mixer_params = mixer.params(spec.mixer, owns_cache)
        for k, d in mixer_params.items():
            out[spec.mixer_prefix + k] = d
        for k, d in feed_forward_class(spec.feed_forward.kind).params(spec.feed_forward).items():
            out[spec.ffn_prefix + k] = d
        out[spec.mixer_norm_name] = norm_class(spec.mixer_norm.kind).params(spec.mixer_norm)["weight"]
        out[spec.ffn_norm_name] = norm_class(spec.ffn_norm.kind).params(spec.ffn_norm)["weight"]
        return out

    def __init__(self, spec: BlockSpec, tensors, ops, dtype):
        self.spec = spec
        self.mixer = mixer_class(spec.mixer.kind)(
            spec.mixer, _sub(tensors, spec.mixer_prefix), ops, dtype)
        self.feed_forward = feed_forward_class(spec.feed_forward.kind)(
            spec.feed_forward, _sub(tensors, spec.ffn_prefix), ops, dtype)
        self.mixer_norm = norm_class(spec.mixer_norm.kind)(
            spec.mixer_norm, {"weight": tensors[spec.mixer_norm_name]}, ops, dtype)
        self.ffn_norm = norm_class(spec.ffn_norm.kind)(
            spec.ffn_norm, {"weight": tensors[spec.ffn_norm_name]}, ops, dtype)

    def forward(self, stream: Stream, ctx, cache) -> Stream:
        normed = self.mixer_norm.add_norm(stream.resid, stream.pending, ctx)
        mixed = self.mixer.forward(normed, ctx, cache)
        normed2 = self.ffn_norm.add_norm(stream.resid, mixed, ctx)
        return Stream(stream.resid, self.feed_forward.forward(normed2, ctx))


register_arrangement("pre_norm", PreNormBlock)
