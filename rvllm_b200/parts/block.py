"""Arrangements: how a block wires its norms, mixer and feed-forward.

"pre_norm": h = x + mixer(norm(x)); out = h + ffn(norm(h)) (the reference's
`Layer::forward`, src/model.rs:556-585), with the reference's optional norms of the
mixer's and the feed-forward's output before each addition (src/model.rs:571, 581;
LFM2 uses neither).  The residual stream is float32; each sub-layer's output stays pending and is
added by the next norm's kernel.
"""
from __future__ import annotations

from .base import (Arrangement, Stream, feed_forward_class, mixer_class, norm_class,
                   register_arrangement)
from .spec import BlockSpec


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class PreNormBlock(Arrangement):
    REQUIRED = ("mixer", "ffn")
    OPTIONAL = ("post_mixer", "post_ffn")

    @staticmethod
    def _check(spec: BlockSpec):
        places = PreNormBlock.REQUIRED + PreNormBlock.OPTIONAL
        for place in PreNormBlock.REQUIRED:
            if place not in spec.norms:
                raise ValueError(f"a pre_norm block needs a norm at {place!r}")
        for place in spec.norms:
            if place not in places:
                raise ValueError(f"a pre_norm block has no place {place!r} for a norm "
                                 f"(places: {', '.join(places)})")

    @staticmethod
    def params(spec: BlockSpec, owns_cache: bool = True):
        """Full tensor names -> declarations for one block."""
        PreNormBlock._check(spec)
        out = {}
        mixer = mixer_class(spec.mixer.kind)
        mixer_params = mixer.params(spec.mixer, owns_cache)
        for k, d in mixer_params.items():
            out[spec.mixer_prefix + k] = d
        for k, d in feed_forward_class(spec.feed_forward.kind).params(spec.feed_forward).items():
            out[spec.ffn_prefix + k] = d
        for norm, name in spec.norms.values():
            out[name] = norm_class(norm.kind).params(norm)["weight"]
        return out

    def __init__(self, spec: BlockSpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.mixer = mixer_class(spec.mixer.kind)(
            spec.mixer, _sub(tensors, spec.mixer_prefix), ops, dtype)
        self.feed_forward = feed_forward_class(spec.feed_forward.kind)(
            spec.feed_forward, _sub(tensors, spec.ffn_prefix), ops, dtype)

        def build(place):
            if place not in spec.norms:
                return None
            norm, name = spec.norms[place]
            return norm_class(norm.kind)(norm, {"weight": tensors[name]}, ops, dtype)

        self.mixer_norm, self.ffn_norm = build("mixer"), build("ffn")
        self.post_mixer, self.post_ffn = build("post_mixer"), build("post_ffn")

    def forward(self, stream: Stream, ctx, cache) -> Stream:
        normed = self.mixer_norm.add_norm(stream.resid, stream.pending, ctx)
        mixed = self.mixer.forward(normed, ctx, cache)
        if self.post_mixer is not None:
            mixed = self.post_mixer.norm(mixed, ctx)
        normed2 = self.ffn_norm.add_norm(stream.resid, mixed, ctx)
        out = self.feed_forward.forward(normed2, ctx)
        if self.post_ffn is not None:
            out = self.post_ffn.norm(out, ctx)
        return Stream(stream.resid, out)


register_arrangement("pre_norm", PreNormBlock)
