"""A second plain LFM2, independent of `plain_lfm2.py`: NumPy, float64, explicit loops.

It is written from the architecture's formulas alone (the layer table: embedding,
pre-norm block with two residuals, RMSNorm with eps inside the root, gated short
convolution with chunks B, C, x and the oldest tap first, grouped-query attention with
per-head q/k RMSNorm before a rotate-half rotation, SwiGLU, final norm and tied or untied
head) and shares no helper with the torch oracle: it has its own reader for the model
folder, its own feed-forward size rule and token-by-token, head-by-head loops where the
other uses tensor operations.  Two independent restatements that agree to 1e-11 (given
the same rotation angles) make a misread formula in either one visible.  The reference's lines for each step are cited in
`plain_lfm2.py`; here only the formulas are stated.

Everything is float64 except the rotation angles, which the architecture defines in
float32 steps (frequency = theta^(-2j/d) by a float32 power, angle = position * frequency
in float32, then cosine and sine in float32): those follow that definition.
"""
import json
import math
import os
import struct

import numpy as np


def _read_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode())
        data = f.read()
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[lo:hi]
        kind = meta["dtype"]
        if kind == "BF16":            # the upper half of a float32
            half = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = half.view(np.float32).astype(np.float64)
        elif kind == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif kind == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif kind == "F64":
            arr = np.frombuffer(raw, dtype="<f8").copy()
        else:
            raise ValueError(f"{name}: dtype {kind} is not handled here")
        tensors[name] = arr.reshape(meta["shape"])
    return cfg, tensors


def _ffn_width(cfg):
    width = int(cfg["block_ff_dim"])
    if cfg.get("block_auto_adjust_ff_dim", True):
        width = (2 * width) // 3
        if cfg.get("block_ffn_dim_multiplier") is not None:
            width = int(cfg["block_ffn_dim_multiplier"] * width)
        step = int(cfg.get("block_multiple_of", 256))
        while width % step:
            width += 1
    return width


def _rms(vec, weight, eps):
    mean_square = 0.0
    for value in vec:
        mean_square += value * value
    mean_square /= len(vec)
    return vec / math.sqrt(mean_square + eps) * weight


def _matvec(matrix, vec, bias=None):
    out = matrix @ vec                  # rows of `matrix` are output channels
    return out if bias is None else out + bias


def _angles(theta, head_dim, position):
    half = head_dim // 2
    cos = np.empty(half)
    sin = np.empty(half)
    for j in range(half):
        freq = np.power(np.float32(theta), np.float32(-2.0 * j) / np.float32(head_dim),
                        dtype=np.float32)
        angle = np.float32(position) * freq
        cos[j] = np.cos(angle, dtype=np.float32)
        sin[j] = np.sin(angle, dtype=np.float32)
    return cos, sin


def _rotate(head, cos, sin):
    half = len(head) // 2
    out = np.empty_like(head)
    for j in range(half):
        a, b = head[j], head[j + half]
        out[j] = a * cos[j] - b * sin[j]
        out[j + half] = a * sin[j] + b * cos[j]
    return out


def _attention_layer(normed, w, p, cfg, table=None):
    n = len(normed)
    heads = cfg["num_attention_heads"]
    kv_heads = cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // heads
    eps = cfg["norm_eps"]
    share = heads // kv_heads
    queries = np.empty((n, heads, d))
    keys = np.empty((n, kv_heads, d))
    values = np.empty((n, kv_heads, d))
    for t in range(n):
        cos, sin = table(t) if table is not None else _angles(cfg["rope_theta"], d, t)
        q = _matvec(w[p + "q_proj.weight"], normed[t]).reshape(heads, d)
        k = _matvec(w[p + "k_proj.weight"], normed[t]).reshape(kv_heads, d)
        values[t] = _matvec(w[p + "v_proj.weight"], normed[t]).reshape(kv_heads, d)
        for h in range(heads):
            queries[t, h] = _rotate(_rms(q[h], w[p + "q_layernorm.weight"], eps), cos, sin)
        for g in range(kv_heads):
            keys[t, g] = _rotate(_rms(k[g], w[p + "k_layernorm.weight"], eps), cos, sin)
    out = np.empty((n, w[p + "out_proj.weight"].shape[0]))
    for t in range(n):
        merged = np.empty(heads * d)
        for h in range(heads):
            g = h // share
            scores = np.array([queries[t, h] @ keys[s, g] for s in range(t + 1)]) / math.sqrt(d)
            weights = np.exp(scores - scores.max())
            weights /= weights.sum()
            acc = np.zeros(d)
            for s in range(t + 1):
                acc += weights[s] * values[s, g]
            merged[h * d:(h + 1) * d] = acc
        out[t] = _matvec(w[p + "out_proj.weight"], merged)
    return out


def _conv_layer(normed, w, p, cfg):
    n = len(normed)
    width = cfg["hidden_size"]
    bias = bool(cfg.get("conv_bias", False))
    filt = w[p + "conv.weight"].reshape(width, -1)
    taps = filt.shape[1]
    gated = []                              # B * x of every position so far
    out = np.empty((n, width))
    for t in range(n):
        row = _matvec(w[p + "in_proj.weight"], normed[t], w[p + "in_proj.bias"] if bias else None)
        b_part, c_part, x_part = row[:width], row[width:2 * width], row[2 * width:]
        gated.append(b_part * x_part)
        acc = np.zeros(width)
        for k in range(taps):               # tap taps-1 meets the token itself, tap 0 the oldest
            src = t - (taps - 1) + k
            if src >= 0:
                acc += filt[:, k] * gated[src]
        if bias:
            acc = acc + w[p + "conv.bias"]
        out[t] = _matvec(w[p + "out_proj.weight"], c_part * acc,
                         w[p + "out_proj.bias"] if bias else None)
    return out


def logits(folder, ids, table=None):
    """float64 logits [len(ids), vocab] of the token sequence `ids`.  `table(position)`, if
    given, supplies (cos, sin) of the rotation instead of `_angles`: two float32 power
    functions may differ in the last bit of a frequency, and a caller that wants to compare
    beyond that hands both implementations the same angles."""
    cfg, w = _read_folder(folder)
    eps = cfg["norm_eps"]
    if "full_attn_idxs" in cfg:
        attention = set(cfg["full_attn_idxs"])
    else:
        attention = {i for i, k in enumerate(cfg["layer_types"]) if k == "full_attention"}
    stream = np.stack([w["model.embed_tokens.weight"][t] for t in ids])
    width_ffn = _ffn_width(cfg)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        normed = np.stack([_rms(r, w[p + "operator_norm.weight"], eps) for r in stream])
        if i in attention:
            mixed = _attention_layer(normed, w, p + "self_attn.", cfg, table)
        else:
            mixed = _conv_layer(normed, w, p + "conv.", cfg)
        stream = stream + mixed
        assert w[p + "feed_forward.w1.weight"].shape[0] == width_ffn
        for t in range(len(ids)):
            z = _rms(stream[t], w[p + "ffn_norm.weight"], eps)
            gate = _matvec(w[p + "feed_forward.w1.weight"], z)
            up = _matvec(w[p + "feed_forward.w3.weight"], z)
            act = gate / (1.0 + np.exp(-gate)) * up
            stream[t] = stream[t] + _matvec(w[p + "feed_forward.w2.weight"], act)
    head = w.get("lm_head.weight")
    if head is None:
        head = w["model.embed_tokens.weight"]
    return np.stack([_matvec(head, _rms(r, w["model.embedding_norm.weight"], eps))
                     for r in stream])
