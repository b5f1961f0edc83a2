"""Plain, slow LFM2 for the tests: whole sequences, no cache, one function per part.

This file is the oracle the engine is compared with. It shares no code with the
product package: it reads ``config.json`` and the safetensors file by itself and
computes every formula with ordinary torch CPU tensor operations.

Where its numbers come from.  The reference project (ermolushka/rvllm) is a Rust
crate whose dependencies are not available offline, so its model code cannot be
compiled or imported for a numeric comparison.  Every function below therefore rests
on the reference's *formulas*; each cites the file and lines it restates.  Three
things that execute hold the formulas in place: the hand-computed vectors of the
reference's own unit tests, restated in ``tests/test_plain.py``; the reference's own
CUDA kernel sources (short convolution, rotation, SiLU gate, RMSNorm, softmax, argmax,
cache write and gather, embedding), compiled as C++ and compared function by function
in ``tests/test_reference_kernels.py`` (their recorded outputs are under
``tests/golden/``); and a second, independent implementation in float64 NumPy,
``tests/plain_numpy64.py``, compared on whole models in ``tests/test_plain.py``.

Options that the reference lacks (convolution biases, the feed-forward size rule)
follow the definitions given in the function that implements them.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch

# ----------------------------------------------------------------------------------
# model folder


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
}


def read_safetensors(path: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """All tensors of a safetensors file, floating ones widened to ``dtype``."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        body = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(body[a:b]), dtype=_ST_DTYPES[meta["dtype"]])
        t = t.reshape(meta["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return out


def feed_forward_size(cfg: dict) -> int:
    """Width of the SwiGLU hidden layer.

    The reference reads an already adjusted ``feed_forward_length``
    (src/weights.rs:276).  A config.json gives ``block_ff_dim`` and the rule that
    produced that number: with ``block_auto_adjust_ff_dim`` take two thirds, apply
    ``block_ffn_dim_multiplier`` if present, then round up to ``block_multiple_of``.
    """
    f = int(cfg["block_ff_dim"])
    if cfg.get("block_auto_adjust_ff_dim", True):
        f = int(2 * f / 3)
        mult = cfg.get("block_ffn_dim_multiplier")
        if mult is not None:
            f = int(mult * f)
        m = int(cfg.get("block_multiple_of", 256))
        f = m * ((f + m - 1) // m)
    return f


def attention_layers(cfg: dict) -> List[int]:
    if "full_attn_idxs" in cfg:
        return list(cfg["full_attn_idxs"])
    return [i for i, k in enumerate(cfg["layer_types"]) if k == "full_attention"]


# ----------------------------------------------------------------------------------
# the parts


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (src/model.rs:200-214)."""
    rms = (x.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt()
    return x / rms * weight


def rope_cos_sin(theta: float, head_dim: int, positions: Sequence[int], dtype):
    """cos and sin of pos * theta^(-2j/head_dim), j < head_dim/2 (src/model.rs:224-246).

    The reference computes the frequencies, the angles and their cosines in f32; so
    does this function, whatever ``dtype`` the result is widened to afterwards.
    """
    half = head_dim // 2
    j = torch.arange(half, dtype=torch.float32)
    freq = torch.pow(torch.tensor(theta, dtype=torch.float32), -2.0 * j / head_dim)
    pos = torch.tensor(list(positions), dtype=torch.float32).unsqueeze(1)
    angles = pos * freq.unsqueeze(0)
    return angles.cos().to(dtype), angles.sin().to(dtype)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half: dimension i pairs with i + head_dim/2 (src/model.rs:252-263).

    x: [..., n, head_dim]; cos, sin: [n, head_dim/2].
    """
    half = x.shape[-1] // 2
    first, second = x[..., :half], x[..., half:]
    return torch.cat([first * cos - second * sin, first * sin + second * cos], dim=-1)


def embed(ids: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """Rows of the table in token order (src/model.rs:275-280)."""
    return table[torch.tensor(list(ids), dtype=torch.long)]


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """x @ weight^T with weight [out, in] (src/model.rs:288-297, 308-314)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + e^-z) (src/cuda/kernels/silu_gate_multiply.cu:1-11)."""
    return z / (1.0 + torch.exp(-z))


def swiglu_ffn(x, gate_w, up_w, down_w) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (src/model.rs:320-335)."""
    return linear(silu(linear(x, gate_w)) * linear(x, up_w), down_w)


def causal_mask(n: int, window: Optional[int], dtype) -> torch.Tensor:
    """0 where key j is visible to query i, -inf elsewhere (src/model.rs:347-372).

    Key j is hidden when j > i, and with a window when j + window <= i.
    """
    i = torch.arange(n).unsqueeze(1)
    j = torch.arange(n).unsqueeze(0)
    hidden = j > i
    if window is not None:
        hidden = hidden | (j + window <= i)
    mask = torch.zeros(n, n, dtype=dtype)
    mask[hidden] = float("-inf")
    return mask


def gqa_attention(q, k, v, mask, scale: Optional[float] = None) -> torch.Tensor:
    """softmax(q k^T / sqrt(head_dim) + mask) v with grouped heads (src/model.rs:377-415).

    q: [heads, n, hd]; k, v: [kv_heads, n, hd]; query heads [g*G, (g+1)*G) use
    key/value head g.  Returns [heads, n, hd].
    """
    heads, n, hd = q.shape
    kv_heads = k.shape[0]
    group = heads // kv_heads
    if scale is None:
        scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    for h in range(heads):
        g = h // group
        scores = (q[h] @ k[g].t()) * scale + mask
        scores = scores - scores.max(dim=-1, keepdim=True).values
        p = torch.exp(scores)
        p = p / p.sum(dim=-1, keepdim=True)
        out[h] = p @ v[g]
    return out


def attention_mixer(normed, w: dict, prefix: str, cfg: dict, window: Optional[int] = None):
    """The attention mixer of one layer over a whole sequence (src/model.rs:591-653).

    Projections without bias, per-head RMSNorm of q and k before the rotation
    (src/model.rs:608-613), rotation of q and k, causal grouped attention, output
    projection.
    """
    n = normed.shape[0]
    nh = cfg["num_attention_heads"]
    nkv = cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg["norm_eps"]
    q = linear(normed, w[prefix + "q_proj.weight"]).reshape(n, nh, hd)
    k = linear(normed, w[prefix + "k_proj.weight"]).reshape(n, nkv, hd)
    v = linear(normed, w[prefix + "v_proj.weight"]).reshape(n, nkv, hd)
    q = rms_norm(q, w[prefix + "q_layernorm.weight"], eps).transpose(0, 1)
    k = rms_norm(k, w[prefix + "k_layernorm.weight"], eps).transpose(0, 1)
    v = v.transpose(0, 1)
    cos, sin = rope_cos_sin(cfg["rope_theta"], hd, range(n), normed.dtype)
    q = rope_apply(q, cos, sin)
    k = rope_apply(k, cos, sin)
    o = gqa_attention(q, k, v, causal_mask(n, window, normed.dtype))
    o = o.transpose(0, 1).reshape(n, nh * hd)
    return linear(o, w[prefix + "out_proj.weight"])


def short_conv(bx: torch.Tensor, filt: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """Causal depthwise convolution from position 0 (src/model.rs:668-686).

    bx: [n, H]; filt: [H, K], oldest tap first: tap K-1 multiplies the token itself
    (src/cuda/kernels/short_conv.cu:39-42).  The K-1 rows before position 0 are zeros
    (src/conv_cache.rs:69-71).  ``bias`` [H], an option the reference does not have,
    is added to the sum.
    """
    n, hidden = bx.shape
    taps = filt.shape[1]
    rows = torch.cat([torch.zeros(taps - 1, hidden, dtype=bx.dtype), bx], dim=0)
    conv = rows[0:n] * filt[:, 0]
    for k in range(1, taps):
        conv = conv + rows[k:k + n] * filt[:, k]
    return conv if bias is None else conv + bias


def short_conv_mixer(normed, w: dict, prefix: str, cfg: dict) -> torch.Tensor:
    """in_proj -> B*x -> causal conv -> C*y -> out_proj (src/model.rs:659-688).

    The projection's three chunks are B, C, x in this order (src/model.rs:663-666).
    With ``conv_bias`` the three biases are added where a linear layer or a
    convolution adds its bias: after in_proj, after the taps, after out_proj.
    """
    hidden = cfg["hidden_size"]
    use_bias = bool(cfg.get("conv_bias", False))
    bcx = linear(normed, w[prefix + "in_proj.weight"],
                 w[prefix + "in_proj.bias"] if use_bias else None)
    b, c, x = bcx[:, :hidden], bcx[:, hidden:2 * hidden], bcx[:, 2 * hidden:]
    filt = w[prefix + "conv.weight"].reshape(hidden, -1)
    y = c * short_conv(b * x, filt, w[prefix + "conv.bias"] if use_bias else None)
    return linear(y, w[prefix + "out_proj.weight"],
                  w[prefix + "out_proj.bias"] if use_bias else None)


def block(x, w: dict, i: int, cfg: dict, is_attention: bool) -> torch.Tensor:
    """h = x + mixer(norm(x)); out = h + ffn(norm(h)) (src/model.rs:556-585)."""
    p = f"model.layers.{i}."
    eps = cfg["norm_eps"]
    normed = rms_norm(x, w[p + "operator_norm.weight"], eps)
    if is_attention:
        mixed = attention_mixer(normed, w, p + "self_attn.", cfg)
    else:
        mixed = short_conv_mixer(normed, w, p + "conv.", cfg)
    h = x + mixed
    normed2 = rms_norm(h, w[p + "ffn_norm.weight"], eps)
    ffn = swiglu_ffn(normed2, w[p + "feed_forward.w1.weight"],
                     w[p + "feed_forward.w3.weight"], w[p + "feed_forward.w2.weight"])
    return h + ffn


def lm_head(x, w: dict, cfg: dict) -> torch.Tensor:
    """Final norm, then the output matrix or the tied table (src/model.rs:725-728;
    src/weights.rs:339-346)."""
    normed = rms_norm(x, w["model.embedding_norm.weight"], cfg["norm_eps"])
    out_w = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(normed, out_w)


def forward(ids: Sequence[int], w: dict, cfg: dict) -> torch.Tensor:
    """Logits [n, vocab] of a whole sequence (src/model.rs:698-735)."""
    x = embed(ids, w["model.embed_tokens.weight"])
    attn = set(attention_layers(cfg))
    for i in range(cfg["num_hidden_layers"]):
        x = block(x, w, i, cfg, i in attn)
    return lm_head(x, w, cfg)


class PlainModel:
    """A model folder read by this file alone."""

    def __init__(self, folder: str, dtype=torch.float32):
        self.cfg = read_config(folder)
        self.w = read_safetensors(os.path.join(folder, "model.safetensors"), dtype)

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        return forward(ids, self.w, self.cfg)

    def greedy(self, prompt: Sequence[int], new_tokens: int) -> List[int]:
        ids = list(prompt)
        for _ in range(new_tokens):
            ids.append(argmax(self.logits(ids)[-1]))
        return ids[len(prompt):]


# ----------------------------------------------------------------------------------
# sampling


def argmax(logits: torch.Tensor) -> int:
    """First maximum wins; NaN never wins; nothing above -inf gives 0
    (src/sampler.rs:68-78)."""
    best, best_value = 0, float("-inf")
    for i, v in enumerate(logits.tolist()):
        if v > best_value:
            best, best_value = i, v
    return best


def sampling_distribution(logits: torch.Tensor, temperature: float, top_p: float):
    """Probabilities after temperature and nucleus filtering, in float64.

    softmax(logits / T) with the maximum subtracted (src/sampler.rs:80-91), then the
    smallest set of most probable tokens whose mass reaches top_p
    (src/sampler.rs:93-117), renormalised.  Tokens that tie with the last kept one
    are kept too.
    """
    z = logits.double() / temperature
    p = torch.exp(z - z.max())
    p = p / p.sum()
    if top_p < 1.0:
        order = torch.argsort(p, descending=True, stable=True)
        cum = torch.cumsum(p[order], 0)
        cut = int((cum >= top_p).nonzero()[0]) if bool((cum >= top_p).any()) else len(p) - 1
        threshold = p[order[cut]]
        p = torch.where(p >= threshold, p, torch.zeros_like(p))
        p = p / p.sum()
    return p
