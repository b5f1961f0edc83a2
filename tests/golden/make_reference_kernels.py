"""Records what the reference project's own kernels compute on fixed inputs.

    python tests/golden/make_reference_kernels.py

writes `tests/golden/reference_kernels.npz`.  The kernels are the unchanged sources of
ermolushka/rvllm under src/cuda/kernels/ (short_conv.cu, rope.cu, silu_gate_multiply.cu,
rmsnorm.cu, softmax.cu, argmax.cu, kv_write.cu, kv_gather.cu, embed_lookup.cu), compiled
as C++ by `tests/ref_kernels.py`; it needs a checkout of the reference (see there).  The
reference's model code is Rust and cannot be built offline, so these kernels are the part
of it that runs here.  `cases()` builds the inputs from seeds, so only outputs are stored.

`tests/test_reference_kernels.py` compares the plain implementation (`tests/plain_lfm2.py`)
with these outputs, and with the kernels run live when a checkout is present.
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

OUT = os.path.join(HERE, "reference_kernels.npz")

CONV_CASES = {          # name: (taps, hidden, tokens in the sequence, new tokens, seed)
    "conv_k3_tail5": (3, 8, 12, 5, 1),
    "conv_k4_from_zero": (4, 6, 9, 9, 2),          # the window before position 0 is zeros
    "conv_k4_single": (4, 6, 10, 1, 3),            # one new token, a full previous window
    "conv_k3_two_tokens": (3, 5, 7, 2, 4),         # fewer new tokens than the window holds
    "conv_k2": (2, 4, 6, 3, 5),
}
ROPE_CASES = {"rope_hd16": (16, 9, 3, 1000000.0, 6), "rope_hd32": (32, 7, 2, 10000.0, 7),
              "rope_hd64": (64, 5, 4, 1000000.0, 8)}      # head_dim, tokens, heads, theta, seed
ATTN_CASES = {"attn_g2": (4, 2, 16, 11, 9), "attn_mqa": (3, 1, 32, 6, 10)}   # heads, kv, hd, n


def conv_inputs(name):
    taps, hidden, total, new, seed = CONV_CASES[name]
    rng = np.random.default_rng(seed)
    proj = rng.standard_normal((total, 3 * hidden)).astype(np.float32)     # B | C | x, all distinct
    filt = rng.standard_normal((hidden, taps)).astype(np.float32)
    return taps, hidden, total, new, proj, filt


def rope_inputs(name):
    hd, n, heads, theta, seed = ROPE_CASES[name]
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, heads, hd)).astype(np.float32)
    return hd, n, heads, theta, x


def attn_inputs(name):
    heads, kv, hd, n, seed = ATTN_CASES[name]
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((heads, n, hd)).astype(np.float32)
    k = rng.standard_normal((kv, n, hd)).astype(np.float32)
    v = rng.standard_normal((kv, n, hd)).astype(np.float32)
    return heads, kv, hd, n, q, k, v


def rope_table(theta, hd, n):
    """cos, sin [n, hd/2] in float32 steps, as src/model.rs:224-246 computes them."""
    half = hd // 2
    j = np.arange(half, dtype=np.float32)
    freq = np.power(np.float32(theta), (np.float32(-2.0) * j / np.float32(hd))).astype(np.float32)
    ang = (np.arange(n, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def cases(ref):
    """{name: output of the reference kernels}."""
    out = {}
    for name in CONV_CASES:
        taps, hidden, total, new, proj, filt = conv_inputs(name)
        bx = ref.short_conv_bx(proj, hidden)
        first = total - new
        window = np.zeros((1, taps - 1 + new, hidden), np.float32)
        lo = first - (taps - 1)
        for r in range(taps - 1 + new):
            if lo + r >= 0:
                window[0, r] = bx[lo + r]
        out[name] = ref.short_conv_filter_gate(window, filt, proj[first:], 1, new)
    # two requests in one launch, each with its own window
    taps, hidden, total, new, proj, filt = conv_inputs("conv_k3_tail5")
    bx = ref.short_conv_bx(proj, hidden)
    q = 3
    window = np.stack([bx[0:taps - 1 + q], bx[4:4 + taps - 1 + q]])
    rows = np.concatenate([proj[taps - 1:taps - 1 + q], proj[4 + taps - 1:4 + taps - 1 + q]])
    out["conv_batch2"] = ref.short_conv_filter_gate(window, filt, rows, 2, q)
    for name in ROPE_CASES:
        hd, n, heads, theta, x = rope_inputs(name)
        cos, sin = rope_table(theta, hd, n)
        out[name] = ref.rope(x.reshape(n * heads, hd), np.repeat(cos, heads, axis=0),
                             np.repeat(sin, heads, axis=0)).reshape(n, heads, hd)
    rng = np.random.default_rng(11)
    g, u = rng.standard_normal((2, 5, 24)).astype(np.float32) * 3
    out["silu_gate"] = ref.silu_gate_multiply(g, u)
    x = rng.standard_normal((5, 96)).astype(np.float32) * 2
    w = (1 + 0.05 * rng.standard_normal(96)).astype(np.float32)
    out["rmsnorm_eps1e-6"] = ref.rmsnorm(x, w, 1e-6)
    out["rmsnorm_eps1e-5"] = ref.rmsnorm(x * 1e-3, w, 1e-5)      # eps matters at this scale
    for name in ATTN_CASES:
        heads, kv, hd, n, q, k, v = attn_inputs(name)
        group = heads // kv
        o = np.empty_like(q)
        for h in range(heads):
            s = (q[h] @ k[h // group].T) * np.float32(1.0 / math.sqrt(hd))
            s = np.where(np.arange(n)[None, :] > np.arange(n)[:, None], -np.inf, s).astype(np.float32)
            o[h] = ref.softmax(s) @ v[h // group]
        out[name] = o
    rows = np.array([[1, 5, 5, 2], [np.nan, 1, 3, 0], [-np.inf] * 4, [2, 2, 2, 2],
                     [-1, -np.inf, -0.5, -0.5]], np.float32)
    out["argmax_rows"] = ref.argmax(rows).astype(np.int64)
    # paged cache: write 10 tokens of one sequence to scattered blocks, read them back
    nkv, hd, bs, blocks = 2, 8, 4, 6
    k = rng.standard_normal((10, nkv, hd)).astype(np.float32)
    v = rng.standard_normal((10, nkv, hd)).astype(np.float32)
    table = np.array([[4, 1, 5]], np.uint32)
    ck = np.zeros((blocks, bs, nkv, hd), np.float32)
    cv = np.zeros_like(ck)
    pos = np.arange(10)
    ref.kv_write(k, v, table[0][pos // bs], pos % bs, ck, cv)
    out["kv_round_trip_k"] = ref.kv_gather(ck, table, 10)
    out["kv_round_trip_v"] = ref.kv_gather(cv, table, 10)
    tab = rng.standard_normal((7, 5)).astype(np.float32)
    out["embed_rows"] = ref.embed_lookup([0, 6, 3, 3, 1], tab)
    return out


if __name__ == "__main__":
    import ref_kernels
    ref = ref_kernels.load()
    if ref is None:
        sys.exit("no checkout of the reference (set RVLLM_REFERENCE_DIR) or no g++")
    got = cases(ref)
    np.savez_compressed(OUT, **got)
    print(f"wrote {OUT}: {len(got)} outputs, {os.path.getsize(OUT)} bytes")
