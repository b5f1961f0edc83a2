"""The plain implementation against the reference project's own kernels.

The reference's elementwise and row kernels (src/cuda/kernels/*.cu of ermolushka/rvllm)
run on the CPU through `tests/ref_kernels.py`.  Their outputs on fixed inputs are recorded
in `tests/golden/reference_kernels.npz` (by `tests/golden/make_reference_kernels.py`); when
a checkout of the reference is present they are also run live and must reproduce the
record.  Each function of `tests/plain_lfm2.py` that restates one of those kernels is
compared with it here, on inputs where a swapped chunk, a reversed filter or a shifted
window gives different numbers: B, C and x are three different random matrices, filters of
2 to 4 taps, windows that start before position 0, inside a sequence and with fewer new
tokens than the window holds, head sizes 16, 32 and 64.
"""
import math
import os
import sys

import numpy as np
import pytest
import torch

import plain_lfm2 as P
import ref_kernels

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_reference_kernels as G       # noqa: E402

TOL = 2e-6          # float32 rounding of sums of a few dozen terms, relative to the largest value


@pytest.fixture(scope="module")
def golden():
    with np.load(G.OUT) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="module")
def live():
    ref = ref_kernels.load()
    return None if ref is None else G.cases(ref)


def check(name, got, golden, live):
    got = np.asarray(got, dtype=np.float64)
    for label, want in (("recorded", golden[name]), ("live", None if live is None else live[name])):
        if want is None:
            continue
        want = np.asarray(want, dtype=np.float64)
        assert got.shape == want.shape, (name, label, got.shape, want.shape)
        scale = max(1.0, float(np.abs(want[np.isfinite(want)]).max()))
        assert float(np.abs(got - want).max()) <= TOL * scale, (name, label)


def test_live_kernels_reproduce_the_record(golden, live):
    if live is None:
        pytest.skip("no checkout of the reference beside the repository (RVLLM_REFERENCE_DIR)")
    assert sorted(live) == sorted(golden)
    for name, want in golden.items():
        np.testing.assert_allclose(live[name], want, rtol=1e-6, atol=1e-6, err_msg=name)


@pytest.mark.parametrize("name", sorted(G.CONV_CASES))
def test_short_conv_rows(name, golden, live):
    """B*x, the window, the taps and the C gate for the last `new` tokens of a sequence:
    `short_conv` over the whole sequence, rows [total-new, total), gated by C."""
    taps, hidden, total, new, proj, filt = G.conv_inputs(name)
    t = torch.from_numpy(proj)
    b, c, x = t[:, :hidden], t[:, hidden:2 * hidden], t[:, 2 * hidden:]
    y = c * P.short_conv(b * x, torch.from_numpy(filt))
    check(name, y[total - new:].numpy(), golden, live)


def test_short_conv_two_requests(golden, live):
    taps, hidden, total, new, proj, filt = G.conv_inputs("conv_k3_tail5")
    t = torch.from_numpy(proj)
    b, c, x = t[:, :hidden], t[:, hidden:2 * hidden], t[:, 2 * hidden:]
    # the recorded launch holds rows [2, 5) of a sequence that starts at row 0 and rows
    # [6, 9) of one that starts at row 4: each window begins with the request's own rows
    first = (c[0:5] * P.short_conv((b * x)[0:5], torch.from_numpy(filt)))[2:5]
    second = (c[4:9] * P.short_conv((b * x)[4:9], torch.from_numpy(filt)))[2:5]
    check("conv_batch2", torch.cat([first, second]).numpy(), golden, live)


@pytest.mark.parametrize("name", sorted(G.CONV_CASES))
def test_short_conv_mixer_chunk_order(name, golden, live):
    """The mixer function itself, with an in_proj that reproduces the recorded projection
    rows: were its three chunks read in another order than B, C, x, or its filter taps
    reversed, the rows would differ from the kernels' output."""
    taps, hidden, total, new, proj, filt = G.conv_inputs(name)
    # normed = identity rows would need total == hidden; instead solve normed . W^T = proj
    rng = np.random.default_rng(100)
    normed = rng.standard_normal((total, total + 3)).astype(np.float64)
    w_in = np.linalg.lstsq(normed, proj.astype(np.float64), rcond=None)[0].T    # [3H, in]
    assert np.abs(normed @ w_in.T - proj).max() < 1e-9
    w = {"p.in_proj.weight": torch.from_numpy(w_in),
         "p.conv.weight": torch.from_numpy(filt.astype(np.float64)).reshape(hidden, 1, taps),
         "p.out_proj.weight": torch.eye(hidden, dtype=torch.float64)}
    out = P.short_conv_mixer(torch.from_numpy(normed), w, "p.", {"hidden_size": hidden})
    check(name, out[total - new:].numpy(), golden, live)


@pytest.mark.parametrize("name", sorted(G.ROPE_CASES))
def test_rope(name, golden, live):
    hd, n, heads, theta, x = G.rope_inputs(name)
    cos, sin = P.rope_cos_sin(theta, hd, range(n), torch.float32)
    got = P.rope_apply(torch.from_numpy(x).transpose(0, 1), cos, sin).transpose(0, 1)
    check(name, got.numpy(), golden, live)


def test_silu_gate(golden, live):
    rng = np.random.default_rng(11)
    g, u = rng.standard_normal((2, 5, 24)).astype(np.float32) * 3
    check("silu_gate", (P.silu(torch.from_numpy(g)) * torch.from_numpy(u)).numpy(), golden, live)


def test_rms_norm(golden, live):
    rng = np.random.default_rng(11)
    rng.standard_normal((2, 5, 24))
    x = torch.from_numpy(rng.standard_normal((5, 96)).astype(np.float32) * 2)
    w = torch.from_numpy((1 + 0.05 * rng.standard_normal(96)).astype(np.float32))
    check("rmsnorm_eps1e-6", P.rms_norm(x, w, 1e-6).numpy(), golden, live)
    check("rmsnorm_eps1e-5", P.rms_norm(x * 1e-3, w, 1e-5).numpy(), golden, live)
    # eps sits inside the square root: at this scale it changes the result by a fifth
    assert float((P.rms_norm(x * 1e-3, w, 1e-5) - P.rms_norm(x * 1e-3, w, 0.0)).abs().max()) > 0.1


@pytest.mark.parametrize("name", sorted(G.ATTN_CASES))
def test_attention_softmax(name, golden, live):
    """Scaled scores, causal mask, the reference's softmax kernel and P.V, against
    `gqa_attention` with `causal_mask`."""
    heads, kv, hd, n, q, k, v = G.attn_inputs(name)
    got = P.gqa_attention(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v),
                          P.causal_mask(n, None, torch.float32))
    check(name, got.numpy(), golden, live)


def test_argmax(golden, live):
    rows = torch.tensor([[1, 5, 5, 2], [math.nan, 1, 3, 0], [-math.inf] * 4, [2, 2, 2, 2],
                         [-1, -math.inf, -0.5, -0.5]], dtype=torch.float32)
    check("argmax_rows", [P.argmax(r) for r in rows], golden, live)


def test_cache_round_trip_and_embedding(golden, live):
    """kv_write then kv_gather give back keys and values in [batch, kv head, position, d]
    order; embed_lookup gives rows in token order like `embed`."""
    rng = np.random.default_rng(11)
    rng.standard_normal((2, 5, 24)); rng.standard_normal((5, 96)); rng.standard_normal(96)
    k = rng.standard_normal((10, 2, 8)).astype(np.float32)
    v = rng.standard_normal((10, 2, 8)).astype(np.float32)
    check("kv_round_trip_k", k.transpose(1, 0, 2)[None], golden, live)
    check("kv_round_trip_v", v.transpose(1, 0, 2)[None], golden, live)
    tab = rng.standard_normal((7, 5)).astype(np.float32)
    check("embed_rows", P.embed([0, 6, 3, 3, 1], torch.from_numpy(tab)).numpy(), golden, live)
