"""Grouped-query attention over a paged cache.

In the reference's order (src/model.rs:591-653): q, k, v projections without bias;
per-head RMSNorm of q and k (src/model.rs:608-613); rotation of q and k; k and v
written into the cache at each token's (page, slot) (src/model.rs:631-640); softmax(q
k^T / sqrt(head_dim)) v over the keys at or before the query's position, query heads
[g*G, (g+1)*G) sharing key/value head g (src/model.rs:377-415); output projection.

What differs by design: q, k and v are one [(heads + 2 kv_heads) * head_dim, hidden]
matrix product; norm, rotation and the cache write are one kernel (for a few tokens: the
product's own epilogue); attention reads
the pages through the block table instead of gathering them into a dense batch
(src/kv_storage.rs:157-173), keeps no score matrix and needs no mask tensor
(src/model.rs:347-372): a key at position j is visible to a query at position p iff
j <= p, and with a window iff j > p - window.

A call whose cache belongs to another call (`cache.owns` false) has no k and v of
its own: it projects q only and reads the other call's pages.
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, PagedNeed, position_class, register_mixer
from .spec import AttentionSpec, ParamDecl


class Attention(Mixer):
    @staticmethod
    def _names(spec):
        n = spec.names
        return {k: n.get(k, k + ".weight") for k in
                ("q_proj", "k_proj", "v_proj", "out_proj", "q_norm", "k_norm")}

    @staticmethod
    def params(spec: AttentionSpec, owns_cache: bool = True):
        n = Attention._names(spec)
        qd, kd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        p = {n["q_proj"]: ParamDecl((qd, spec.hidden), "linear"),
             n["out_proj"]: ParamDecl((spec.hidden, qd), "linear")}
        if owns_cache:
            p[n["k_proj"]] = ParamDecl((kd, spec.hidden), "linear")
            p[n["v_proj"]] = ParamDecl((kd, spec.hidden), "linear")
        if spec.qk_norm is not None:
            p[n["q_norm"]] = ParamDecl((spec.head_dim,), "norm")
            if owns_cache:
                p[n["k_norm"]] = ParamDecl((spec.head_dim,), "norm")
        return p

    @staticmethod
    def cache_need(spec: AttentionSpec):
        return PagedNeed(spec.num_kv_heads, spec.head_dim, spec.window)

    @staticmethod
    def workspace_bytes(spec: AttentionSpec, ops, max_requests: int, max_context: int) -> int:
        sizer = getattr(ops, "attention_scratch_bytes", None)
        if sizer is None:
            return 0
        return sizer(max_requests, spec.num_heads, spec.head_dim, max_context)

    def __init__(self, spec: AttentionSpec, tensors, ops, dtype):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"invalid attention head counts: {spec.num_heads} query, "
                             f"{spec.num_kv_heads} KV")
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        q = tensors[n["q_proj"]]
        self.has_kv = n["k_proj"] in tensors
        if self.has_kv:
            self.w_qkv = torch.cat([q, tensors[n["k_proj"]].to(q.dtype),
                                    tensors[n["v_proj"]].to(q.dtype)], dim=0).contiguous()
        else:
            self.w_qkv = q.contiguous()
        self.w_q = self.w_qkv[:spec.num_heads * spec.head_dim]
        self.w_out = tensors[n["out_proj"]].contiguous()
        self.q_norm = self.k_norm = None
        if spec.qk_norm is not None:
            self.q_norm = tensors[n["q_norm"]].to(torch.float32).contiguous()
            if self.has_kv:
                self.k_norm = tensors[n["k_norm"]].to(torch.float32).contiguous()
        self.position = position_class(spec.position.kind)(spec.position, q.device)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)

    def forward(self, normed, ctx, cache):
        s = self.spec
        owns = cache.owns
        if owns and not self.has_kv:
            raise ValueError("attention: this call owns a cache but the block has no "
                             "key and value projections")
        group = ctx.groups[cache.group]
        qkv = self.ops.linear_qk_norm_rope_write(
            normed, self.w_qkv if owns else self.w_q, s.num_heads,
            s.num_kv_heads if owns else 0, s.head_dim,
            self.q_norm, self.k_norm if owns else None, s.qk_norm.eps if s.qk_norm else 0.0,
            self.position.rotation_table(), ctx.positions, group.slot_mapping,
            cache.k if owns else None, cache.v if owns else None, out_dtype=self.dtype)
        out = self.ops.new_rows(normed.shape[0], s.num_heads * s.head_dim, self.dtype, normed.device)
        self.ops.paged_attention(qkv, s.num_heads, s.num_kv_heads, s.head_dim,
                                 cache.k, cache.v, ctx, group, self.scale, s.window, out)
        return self.ops.linear(out, self.w_out, out_dtype=self.dtype)


register_mixer("attention", Attention)
