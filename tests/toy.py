"""A toy architecture defined entirely in the tests, to show that parts and
architectures plug in without touching the package:

* `ToyDecay`, a mixer with a state of its own (one float32 vector per request):
  s_t = decay * s_{t-1} + W x_t, out_t = s_t; it relies on the cache manager's promise
  that a slot is zero when a request receives it, and its weight asks the random-weights
  mode for a distribution of its own;
* `ScaledRelu`, another feed-forward: down(relu(up(x)) * gain);
* `SoftRouted`, a feed-forward with a router: float32 router logits, softmax gates over
  its experts, out = sum_e gate_e * down_e(relu(up_e(x))) (every expert weighted, so the
  result is continuous in the logits and a test cannot flip on a near-tie);
* `HalfRope`, another position encoding: the reference rotation at half the angle;
* "ToyForCausalLM": blocks [decay, windowed attention with HalfRope, attention without
  position encoding or q/k norm and a custom scale, decay with the routed feed-forward and
  norms after the mixer and after the feed-forward as well as before them],
  run in the order
  0, 1, 2, 1(reading nothing: a second call with its own cache), 3, 2(reading the cache
  of the first call of block 2), so a block runs twice and a call reads another call's
  cache.

It is not a model of anyone's; `toy_plain_logits` is its plain whole-sequence forward.
"""
import math
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional

import torch

import plain_lfm2 as P
from rvllm_b200.config import register_architecture
from rvllm_b200.config.base import Reader
from rvllm_b200.parts import (AttentionSpec, BlockSpec, FeedForward, LayerCall, Mixer, ModelSpec,
                              NormSpec, ParamDecl, PositionEncoding, PositionSpec, StateNeed,
                              register_feed_forward, register_mixer, register_position)
from rvllm_b200.parts.spec import FeedForwardSpec, MixerSpec


# ---- parts -----------------------------------------------------------------------------

@dataclass(frozen=True)
class ToyDecaySpec(MixerSpec):
    decay: float = 0.5


class ToyDecay(Mixer):
    @staticmethod
    def params(spec, owns_cache=True):
        # a distribution of its own for the random-weights mode
        return {"w.weight": ParamDecl((spec.hidden, spec.hidden), "normal", mean=0.0, std=0.03)}

    @staticmethod
    def cache_need(spec):
        return StateNeed((spec.hidden,))

    def __init__(self, spec, tensors, ops, dtype):
        self.spec, self.ops, self.dtype = spec, ops, dtype
        self.w = tensors["w.weight"]

    def forward(self, normed, ctx, cache):
        y = self.ops.linear(normed, self.w, out_dtype=torch.float32)
        out = torch.empty_like(y)
        starts = ctx.q_start.tolist()
        slots = ctx.state_slot.tolist()
        for r in range(ctx.n_reqs):
            if slots[r] < 0:
                continue
            # no test of "is this the request's first step": the cache manager hands out a
            # slot cleared to zero, so the state before position 0 is simply what is there
            s = cache.state[slots[r]]
            for t in range(starts[r], starts[r + 1]):
                s = self.spec.decay * s + y[t]
                out[t] = s
            cache.state[slots[r]] = s
        return out.to(self.dtype)


@dataclass(frozen=True)
class ScaledReluSpec(FeedForwardSpec):
    width: int = 0
    gain: float = 1.0


class ScaledRelu(FeedForward):
    @staticmethod
    def params(spec):
        return {"up.weight": ParamDecl((spec.width, spec.hidden), "linear"),
                "down.weight": ParamDecl((spec.hidden, spec.width), "linear")}

    def __init__(self, spec, tensors, ops, dtype):
        self.spec, self.ops, self.dtype = spec, ops, dtype
        self.up, self.down = tensors["up.weight"], tensors["down.weight"]

    def forward(self, normed, ctx):
        h = torch.relu(self.ops.linear(normed, self.up, out_dtype=self.dtype)) * self.spec.gain
        return self.ops.linear(h.to(self.dtype), self.down, out_dtype=self.dtype)


@dataclass(frozen=True)
class SoftRoutedSpec(FeedForwardSpec):
    width: int = 0
    experts: int = 2


class SoftRouted(FeedForward):
    @staticmethod
    def params(spec):
        p = {"router.weight": ParamDecl((spec.experts, spec.hidden), "linear")}
        for e in range(spec.experts):
            p[f"experts.{e}.up.weight"] = ParamDecl((spec.width, spec.hidden), "linear")
            p[f"experts.{e}.down.weight"] = ParamDecl((spec.hidden, spec.width), "linear")
        return p

    def __init__(self, spec, tensors, ops, dtype):
        self.spec, self.ops, self.dtype = spec, ops, dtype
        self.router = tensors["router.weight"]
        self.up = [tensors[f"experts.{e}.up.weight"] for e in range(spec.experts)]
        self.down = [tensors[f"experts.{e}.down.weight"] for e in range(spec.experts)]

    def forward(self, normed, ctx):
        gates = torch.softmax(self.ops.linear(normed, self.router, out_dtype=torch.float32), dim=-1)
        out = torch.zeros((normed.shape[0], self.spec.hidden), dtype=torch.float32,
                          device=normed.device)
        for e in range(self.spec.experts):
            h = torch.relu(self.ops.linear(normed, self.up[e], out_dtype=self.dtype))
            out += gates[:, e:e + 1] * self.ops.linear(h, self.down[e], out_dtype=torch.float32)
        return out.to(self.dtype)


class HalfRope(PositionEncoding):
    def __init__(self, spec, device):
        half = spec.head_dim // 2
        j = torch.arange(half, dtype=torch.float32)
        freq = torch.pow(torch.tensor(spec.theta, dtype=torch.float32), -2.0 * j / spec.head_dim)
        ang = 0.5 * torch.arange(spec.max_position, dtype=torch.float32).unsqueeze(1) * freq
        self.table = (ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous())

    def rotation_table(self):
        return self.table


# ---- the architecture ----------------------------------------------------------------------

@dataclass(frozen=True)
class ToyConfig:
    architecture: str
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    width: int
    vocab_size: int
    max_position: int
    eps: float
    window: int
    theta: float
    decay: float
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, data, where="config.json"):
        r = Reader(data, where)
        return cls(r.str_list("architectures")[0], r.int("hidden"), r.int("heads"),
                   r.int("kv_heads"), r.int("head_dim"), r.int("width"), r.int("vocab_size"),
                   r.int("max_position"), r.float("eps"), r.int("window"), r.float("theta"),
                   r.float("decay"), r.str("torch_dtype", "bfloat16"))

    def to_dict(self):
        d = dict(self.__dict__)
        d["architectures"] = [d.pop("architecture")]
        return d


TOY = {"architectures": ["ToyForCausalLM"], "hidden": 48, "heads": 6, "kv_heads": 2, "head_dim": 16,
       "width": 80, "vocab_size": 300, "max_position": 256, "eps": 1e-5, "window": 9,
       "theta": 500.0, "decay": 0.6, "torch_dtype": "bfloat16"}
ORDER = [(0, None), (1, None), (2, None), (1, None), (3, None), (2, 2)]   # (block, cache_of)


def toy_spec(cfg: ToyConfig) -> ModelSpec:
    norm = NormSpec("rmsnorm", cfg.hidden, cfg.eps)
    ffn = ScaledReluSpec("toy_scaled_relu", cfg.hidden, width=cfg.width, gain=1.25)
    decay = ToyDecaySpec("toy_decay", cfg.hidden, decay=cfg.decay)
    local = AttentionSpec("attention", cfg.hidden, num_heads=cfg.heads, num_kv_heads=cfg.kv_heads,
                          head_dim=cfg.head_dim, qk_norm=NormSpec("rmsnorm", cfg.head_dim, cfg.eps),
                          position=PositionSpec("toy_half_rope", cfg.head_dim, cfg.theta,
                                                cfg.max_position), window=cfg.window)
    plain = AttentionSpec("attention", cfg.hidden, num_heads=cfg.heads, num_kv_heads=cfg.kv_heads,
                          head_dim=cfg.head_dim, qk_norm=None, position=PositionSpec("none"),
                          window=None, scale=0.3)
    routed = SoftRoutedSpec("toy_soft_routed", cfg.hidden, width=cfg.width // 2, experts=3)
    layers = []
    for i, mixer in enumerate([decay, local, plain, decay]):
        p = f"blocks.{i}."
        norms = {"mixer": (norm, p + "norm1.weight"), "ffn": (norm, p + "norm2.weight")}
        if i == 3:      # this block also normalises what its mixer and feed-forward give back
            norms["post_mixer"] = (norm, p + "post1.weight")
            norms["post_ffn"] = (norm, p + "post2.weight")
        layers.append(BlockSpec("pre_norm", mixer, routed if i == 3 else ffn, norms,
                                p + "mixer.", p + "ffn."))
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden=cfg.hidden,
                     max_position=cfg.max_position, layers=tuple(layers),
                     order=tuple(LayerCall(b, c) for b, c in ORDER), final_norm=norm,
                     embedding_name="embed.weight", final_norm_name="norm.weight",
                     head_name="head.weight")


def register_toy():
    register_mixer("toy_decay", ToyDecay, replace=True)
    register_feed_forward("toy_scaled_relu", ScaledRelu, replace=True)
    register_feed_forward("toy_soft_routed", SoftRouted, replace=True)
    register_position("toy_half_rope", HalfRope, replace=True)
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec, replace=True)


# ---- its plain forward ---------------------------------------------------------------------

def toy_plain_logits(ids, w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """Whole sequence, no cache; w holds float32 tensors by file name."""
    H, nh, nkv, hd, eps = cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["eps"]
    n = len(ids)
    x = P.embed(ids, w["embed.weight"])
    kv_of_call = {}

    def ffn(h, p):
        if p + "router.weight" in w:
            gates = torch.softmax(P.linear(h, w[p + "router.weight"]), dim=-1)
            out = torch.zeros(h.shape[0], H)
            for e in range(gates.shape[1]):
                q = p + f"experts.{e}."
                out = out + gates[:, e:e + 1] * P.linear(torch.relu(P.linear(h, w[q + "up.weight"])),
                                                         w[q + "down.weight"])
            return out
        return P.linear(torch.relu(P.linear(h, w[p + "up.weight"])) * 1.25, w[p + "down.weight"])

    for call, (b, cache_of) in enumerate(ORDER):
        p = f"blocks.{b}."
        normed = P.rms_norm(x, w[p + "norm1.weight"], eps)
        if b in (0, 3):
            y = P.linear(normed, w[p + "mixer.w.weight"])
            s, rows = torch.zeros(H), []
            for t in range(n):
                s = cfg["decay"] * s + y[t]
                rows.append(s)
            mixed = torch.stack(rows)
        else:
            m = p + "mixer."
            q = P.linear(normed, w[m + "q_proj.weight"]).reshape(n, nh, hd)
            if b == 1:
                q = P.rms_norm(q, w[m + "q_norm.weight"], eps)
            if cache_of is None:
                k = P.linear(normed, w[m + "k_proj.weight"]).reshape(n, nkv, hd)
                v = P.linear(normed, w[m + "v_proj.weight"]).reshape(n, nkv, hd)
                if b == 1:
                    k = P.rms_norm(k, w[m + "k_norm.weight"], eps)
            q = q.transpose(0, 1)
            if b == 1:
                half = hd // 2
                j = torch.arange(half, dtype=torch.float32)
                freq = torch.pow(torch.tensor(cfg["theta"], dtype=torch.float32), -2.0 * j / hd)
                ang = 0.5 * torch.arange(n, dtype=torch.float32).unsqueeze(1) * freq
                q = P.rope_apply(q, ang.cos(), ang.sin())
                if cache_of is None:
                    k = P.rope_apply(k.transpose(0, 1), ang.cos(), ang.sin()).transpose(0, 1)
            if cache_of is None:
                kv_of_call[call] = (k.transpose(0, 1), v.transpose(0, 1))
                kk, vv = kv_of_call[call]
            else:
                kk, vv = kv_of_call[cache_of]
            window = cfg["window"] if b == 1 else None
            scale = None if b == 1 else 0.3
            o = P.gqa_attention(q, kk, vv, P.causal_mask(n, window, torch.float32), scale)
            mixed = P.linear(o.transpose(0, 1).reshape(n, nh * hd), w[m + "out_proj.weight"])
        if p + "post1.weight" in w:
            mixed = P.rms_norm(mixed, w[p + "post1.weight"], eps)
        h = x + mixed
        out = ffn(P.rms_norm(h, w[p + "norm2.weight"], eps), p + "ffn.")
        if p + "post2.weight" in w:
            out = P.rms_norm(out, w[p + "post2.weight"], eps)
        x = h + out
    return P.linear(P.rms_norm(x, w["norm.weight"], eps), w["head.weight"])
