"""The generic model: embedding, the blocks in their run order, final norm and head.

It executes a `ModelSpec` and knows no architecture.  In the reference this is
`Model::hidden` / `lm_head` / `forward_last` (src/model.rs:698-745): embed, run the
layers, keep only the rows whose logits are wanted, final norm, output matrix (the
embedding table when the model has no head of its own, src/weights.rs:339-346).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import Stream, arrangement_class, mixer_class, norm_class
from .spec import ModelSpec, ParamDecl


def block_owns_cache(spec: ModelSpec) -> List[bool]:
    """For each block: does any of its calls own a cache (rather than read another's)?"""
    owns = [False] * len(spec.layers)
    for call in spec.order:
        if call.cache_of is None:
            owns[call.layer] = True
    return owns


def param_decls(spec: ModelSpec) -> Dict[str, ParamDecl]:
    """Every tensor the model reads, by its name in the file."""
    out: Dict[str, ParamDecl] = {
        spec.embedding_name: ParamDecl((spec.vocab_size, spec.hidden), "embedding"),
        spec.final_norm_name: norm_class(spec.final_norm.kind).params(spec.final_norm)["weight"],
    }
    if spec.head_name is not None:
        out[spec.head_name] = ParamDecl((spec.vocab_size, spec.hidden), "linear")
    used = {call.layer for call in spec.order}
    for i, (b, owns) in enumerate(zip(spec.layers, block_owns_cache(spec))):
        if i in used:
            out.update(arrangement_class(b.arrangement).params(b, owns))
    return out


def validate_order(spec: ModelSpec) -> None:
    for pos, call in enumerate(spec.order):
        if not 0 <= call.layer < len(spec.layers):
            raise ValueError(f"run order entry {pos} names layer {call.layer}, "
                             f"but the model has {len(spec.layers)} layers")
        if call.cache_of is not None:
            if not 0 <= call.cache_of < pos:
                raise ValueError(f"run order entry {pos} reads the cache of entry "
                                 f"{call.cache_of}, which does not run before it")
            src = spec.order[call.cache_of]
            if src.cache_of is not None:
                raise ValueError(f"run order entry {pos} reads the cache of entry "
                                 f"{call.cache_of}, which owns none")
            a = mixer_class(spec.layers[call.layer].mixer.kind).cache_need(
                spec.layers[call.layer].mixer)
            b = mixer_class(spec.layers[src.layer].mixer.kind).cache_need(
                spec.layers[src.layer].mixer)
            if a != b:
                raise ValueError(f"run order entry {pos} reads the cache of entry "
                                 f"{call.cache_of}, whose cache has another shape")


class Model:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], ops, dtype):
        validate_order(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        self.embedding = tensors[spec.embedding_name].contiguous()
        self.head = (tensors[spec.head_name].contiguous() if spec.head_name is not None
                     else self.embedding)
        self.final_norm = norm_class(spec.final_norm.kind)(
            spec.final_norm, {"weight": tensors[spec.final_norm_name]}, ops, dtype)
        used = {call.layer for call in spec.order}
        self.blocks = [arrangement_class(b.arrangement)(b, tensors, ops, dtype)
                       if i in used else None for i, b in enumerate(spec.layers)]
        self.device = self.embedding.device

    def cache_needs(self) -> List[Optional[object]]:
        """What each call of the run order has to remember (None: nothing of its own)."""
        needs = []
        for call in self.spec.order:
            m = self.spec.layers[call.layer].mixer
            needs.append(None if call.cache_of is not None
                         else mixer_class(m.kind).cache_need(m))
        return needs

    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the step's tokens; float32 logits [len(ctx.logit_rows), vocab]."""
        n = ctx.n_tokens
        resid = torch.empty((n, self.spec.hidden), dtype=torch.float32, device=self.device)
        self.ops.embed(self.embedding, ctx.token_ids, resid, self.spec.embedding_scale)
        stream = Stream(resid, None)
        for call, cache in zip(self.spec.order, caches):
            stream = self.blocks[call.layer].forward(stream, ctx, cache)
        if ctx.logit_rows.shape[0] == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32,
                               device=self.device)
        normed = self.final_norm.add_norm(stream.resid, stream.pending, ctx,
                                          rows=ctx.logit_rows)
        return self.ops.linear(normed, self.head, out_dtype=torch.float32)
