"""The plain implementation against the reference's own hand-computed vectors (its unit
tests in src/model.rs and src/sampler.rs, restated), and against itself in float64."""
import math

import pytest
import torch

import plain_lfm2 as P
from tiny import write_tiny


def close(got, want, tol):
    assert all(abs(a - b) < tol for a, b in zip(got, want)), (got, want)


def test_rms_norm_hand_computed():
    # src/model.rs:758-775: x = [1,2,3], eps 1e-5 -> [0.46292, 0.92583, 1.38875]
    out = P.rms_norm(torch.tensor([[1.0, 2.0, 3.0]]), torch.ones(3), 1e-5)
    close(out.flatten().tolist(), [0.46292, 0.92583, 1.38875], 1e-4)


def test_rope_position_zero_is_identity():
    # src/model.rs:778-788
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    cos, sin = P.rope_cos_sin(10000.0, 4, [0], torch.float32)
    close(P.rope_apply(x, cos, sin).flatten().tolist(), [1, 2, 3, 4], 1e-6)


def test_rope_position_one_hand_computed():
    # src/model.rs:790-808: theta = [1, 0.01]; (1,0) pairs rotate by 1 and 0.01
    x = torch.tensor([[1.0, 1.0, 0.0, 0.0], [1.0, 1.0, 0.0, 0.0]])
    cos, sin = P.rope_cos_sin(10000.0, 4, [0, 1], torch.float32)
    out = P.rope_apply(x, cos, sin)
    close(out[1].tolist(), [math.cos(1), math.cos(0.01), math.sin(1), math.sin(0.01)], 1e-6)


def test_embed_rows_in_order():
    # src/model.rs:826-841
    table = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    assert P.embed([0, 2, 1], table).flatten().tolist() == [1, 2, 5, 6, 3, 4]


def test_swiglu_identity_weights():
    # src/model.rs:844-863: [silu(1)*1, silu(2)*2] = [0.731059, 3.523188]
    eye = torch.eye(2)
    out = P.swiglu_ffn(torch.tensor([[1.0, 2.0]]), eye, eye, eye)
    close(out.flatten().tolist(), [0.731059, 3.523188], 1e-5)


def test_linear_manual():
    # src/model.rs:866-877
    w = torch.tensor([[1.0, 2, 3], [4, 5, 6]])
    x = torch.tensor([[1.0, 0, 1], [0, 1, 0]])
    assert P.linear(x, w).flatten().tolist() == [4, 10, 2, 5]


def test_gqa_attention_hand_computed():
    # src/model.rs:880-923: two query heads share one KV head; causal
    k = torch.tensor([[[1.0, 0.0], [0.0, 1.0]]])
    v = torch.tensor([[[10.0, 0.0], [0.0, 20.0]]])
    q = torch.tensor([[[1.0, 0.0], [1.0, 0.0]], [[0.0, 1.0], [0.0, 1.0]]])
    out = P.gqa_attention(q, k, v, P.causal_mask(2, None, torch.float32))
    close(out.flatten().tolist(), [10, 0, 6.698, 6.604, 10, 0, 3.302, 13.396], 1e-2)


def test_window_mask():
    # src/model.rs:361-363: key j hidden when j > i or j + window <= i
    m = P.causal_mask(5, 2, torch.float32)
    vis = [[j for j in range(5) if m[i, j] == 0] for i in range(5)]
    assert vis == [[0], [0, 1], [1, 2], [2, 3], [3, 4]]


def test_short_conv_hand_computed():
    # src/model.rs:1261-1288: B = C = x = input, filter [1, 10, 100] oldest first,
    # inputs [1, 2, 3]: conv of x^2 = [100, 410, 941], times x = [100, 820, 2823]
    x = torch.tensor([[1.0], [2.0], [3.0]])
    conv = P.short_conv(x * x, torch.tensor([[1.0, 10.0, 100.0]]))
    assert (x * conv).flatten().tolist() == [100.0, 820.0, 2823.0]
    w = {"p.in_proj.weight": torch.ones(3, 1), "p.conv.weight": torch.tensor([[[1.0, 10.0, 100.0]]]),
         "p.out_proj.weight": torch.ones(1, 1)}
    out = P.short_conv_mixer(x, w, "p.", {"hidden_size": 1})
    assert out.flatten().tolist() == [100.0, 820.0, 2823.0]


def test_argmax_ties_and_nan():
    # src/sampler.rs:146-154 and argmax.cu:1-4
    assert P.argmax(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1
    assert P.argmax(torch.tensor([float("nan"), 1.0, 3.0])) == 2
    assert P.argmax(torch.tensor([float("-inf")] * 3)) == 0


def test_feed_forward_sizes_of_the_published_configs():
    def ff(dim, mult=256, auto=True):
        return P.feed_forward_size({"block_ff_dim": dim, "block_auto_adjust_ff_dim": auto,
                                    "block_multiple_of": mult})
    assert (ff(12288), ff(6656), ff(10240), ff(384, 128), ff(192, 256, False)) == \
        (8192, 4608, 6912, 256, 192)


@pytest.mark.parametrize("name", ["A", "B"])
def test_agrees_with_the_independent_numpy_implementation(tmp_path, name):
    """`plain_numpy64.py` restates the architecture a second time, in float64 NumPy with
    loops and its own reader of the model folder.  Given the same rotation angles the two
    agree to 1e-11 of the largest logit; with each one's own float32 angle table to 1e-7
    (two float32 power functions may differ in the last bit of a frequency, which moves an
    angle by position * 6e-8 relative)."""
    import plain_numpy64
    folder = write_tiny(str(tmp_path), name)
    ids = [(7 * i + 3) % 500 for i in range(40)]
    a = P.PlainModel(folder, torch.float64).logits(ids).numpy()
    scale = float(abs(a).max())
    own = plain_numpy64.logits(folder, ids)
    assert float(abs(a - own).max()) <= 1e-7 * scale
    cfg = P.read_config(folder)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    cos, sin = P.rope_cos_sin(cfg["rope_theta"], hd, range(len(ids)), torch.float64)
    same = plain_numpy64.logits(folder, ids, table=lambda t: (cos[t].numpy(), sin[t].numpy()))
    assert float(abs(a - same).max()) <= 1e-11 * scale
    assert (a.argmax(-1) == same.argmax(-1)).all()


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_agrees_with_float64(tmp_path, name):
    folder = write_tiny(str(tmp_path), name)
    ids = [(7 * i + 3) % 500 for i in range(40)]
    a = P.PlainModel(folder, torch.float32).logits(ids)
    b = P.PlainModel(folder, torch.float64).logits(ids)
    assert float((a.double() - b).abs().max()) <= 2e-6 * float(b.abs().max())


def test_nucleus_keeps_smallest_prefix():
    p = P.sampling_distribution(torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05])), 1.0, 0.75)
    close(p.tolist(), [0.625, 0.375, 0, 0], 1e-6)   # the logs are float32
