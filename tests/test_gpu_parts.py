"""Each part alone on the GPU against the plain formula, and the toy architecture of
tests/toy.py (parts defined outside the package) stepped by the engine on the GPU."""
import math
import os
import random

import pytest
import torch

import plain_lfm2 as P
import schedules
import toy
from rvllm_b200.cache import CacheManager
from rvllm_b200.config import config_from_dict
from rvllm_b200.engine import BatchBuilder, ModelRunner, StepEntry, load_model, make_cache
from rvllm_b200.parts import (AttentionSpec, BlockSpec, NormSpec, PositionSpec, ShortConvSpec,
                              Stream, SwiGLUSpec, arrangement_class, feed_forward_class,
                              mixer_class, norm_class)
from rvllm_b200.weights import write_random_model
from rvllm_b200.weights.random_init import random_tensor

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from rvllm_b200.kernels import cuda_ops
    return cuda_ops()


def bound(dtype):
    return 1e-5 if dtype == torch.float32 else 3e-2


def tensors_for(decls, dtype, seed=0):
    """bfloat16-representable random tensors: (device copies in dtype, float32 host copies)."""
    host = {n: random_tensor(n, d, seed, torch.bfloat16) for n, d in decls.items()}
    return ({n: t.to("cuda", dtype) for n, t in host.items()},
            {n: t.float() for n, t in host.items()})


def context(ops, need, page, lengths, cuts):
    """A cache for one call with `need`, and step contexts that feed each request of
    `lengths` tokens in portions given by `cuts` (cycled)."""
    cache = CacheManager([need], [None], page, 64, len(lengths), dtype=cuts["dtype"], device="cuda")
    builder = BatchBuilder(cache, ops, "cuda", pinned=True)
    for i in range(len(lengths)):
        cache.add(i)
    done = [0] * len(lengths)
    k = 0
    while any(d < n for d, n in zip(done, lengths)):
        entries = []
        for i, n in enumerate(lengths):
            if done[i] < n:
                take = min(cuts["sizes"][k % len(cuts["sizes"])], n - done[i])
                k += 1
                entries.append((i, done[i], take))
        entries.sort(key=lambda e: e[2] != 1)
        for i, a, take in entries:
            cache.reserve(i, a + take)
        ctx = builder.build([StepEntry(i, [0] * take, ()) for i, a, take in entries])
        yield cache, ctx, entries
        for i, a, take in entries:
            cache.advance(i, a + take)
            done[i] = a + take


def check(got, want, dtype):
    err = float((got.float().cpu() - want).abs().max()) / max(1e-6, float(want.abs().max()))
    assert err <= bound(dtype), err


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(ops, dtype):
    spec = NormSpec("rmsnorm", 200, 1e-6)
    cls = norm_class("rmsnorm")
    dev, host = tensors_for(cls.params(spec), dtype)
    part = cls(spec, dev, ops, dtype)
    g = torch.Generator().manual_seed(0)
    resid, delta = torch.randn(9, 200, generator=g), torch.randn(9, 200, generator=g).bfloat16().float()
    r = resid.cuda()
    out = part.add_norm(r, delta.to("cuda", dtype), None)
    check(out, P.rms_norm(resid + delta, host["weight"], 1e-6), dtype)
    check(r, resid + delta, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(ops, dtype):
    spec = SwiGLUSpec("swiglu", 72, ffn_dim=200, names={"gate": "w1.weight", "up": "w3.weight",
                                                         "down": "w2.weight"})
    cls = feed_forward_class("swiglu")
    dev, host = tensors_for(cls.params(spec), dtype)
    part = cls(spec, dev, ops, dtype)
    x = (torch.randn(11, 72, generator=torch.Generator().manual_seed(1)) * 3).bfloat16().float()
    out = part.forward(x.to("cuda", dtype), None)
    check(out, P.swiglu_ffn(x, host["w1.weight"], host["w3.weight"], host["w2.weight"]), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,bias", [(3, False), (4, True)])
def test_short_conv_part_in_portions(ops, dtype, taps, bias):
    hidden = 72
    spec = ShortConvSpec("short_conv", hidden, taps=taps, bias=bias)
    cls = mixer_class("short_conv")
    dev, host = tensors_for(cls.params(spec), dtype)
    part = cls(spec, dev, ops, dtype)
    lengths = [37, 5, 1, 20]
    g = torch.Generator().manual_seed(2)
    xs = [(torch.randn(n, hidden, generator=g) * 2).bfloat16().float() for n in lengths]
    cfg = {"hidden_size": hidden, "conv_bias": bias}
    want = [P.short_conv_mixer(x, {"p." + k: v for k, v in host.items()}, "p.", cfg) for x in xs]
    got = [torch.zeros(n, hidden) for n in lengths]
    for cache, ctx, entries in context(ops, cls.cache_need(spec), 8, lengths,
                                       {"dtype": dtype, "sizes": [2, 7, 1, 3, 16]}):
        x = torch.cat([xs[i][a:a + take] for i, a, take in entries]).to("cuda", dtype)
        y = part.forward(x, ctx, cache.views()[0]).float().cpu()
        at = 0
        for i, a, take in entries:
            got[i][a:a + take] = y[at:at + take]
            at += take
    for g_, w_ in zip(got, want):
        check(g_, w_, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 11])
def test_attention_part_in_portions(ops, dtype, window):
    hidden, nh, nkv, hd = 80, 6, 2, 48
    spec = AttentionSpec("attention", hidden, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                         qk_norm=NormSpec("rmsnorm", hd, 1e-5),
                         position=PositionSpec("rope", hd, 10000.0, 128), window=window,
                         names={"q_norm": "q_layernorm.weight", "k_norm": "k_layernorm.weight"})
    cls = mixer_class("attention")
    dev, host = tensors_for(cls.params(spec), dtype)
    part = cls(spec, dev, ops, dtype)
    lengths = [50, 9, 1, 33]
    g = torch.Generator().manual_seed(3)
    xs = [(torch.randn(n, hidden, generator=g) * 2).bfloat16().float() for n in lengths]
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "norm_eps": 1e-5,
           "rope_theta": 10000.0, "hidden_size": hidden}
    want = [P.attention_mixer(x, {"p." + k: v for k, v in host.items()}, "p.", cfg, window)
            for x in xs]
    got = [torch.zeros(n, hidden) for n in lengths]
    for cache, ctx, entries in context(ops, cls.cache_need(spec), 8, lengths,
                                       {"dtype": dtype, "sizes": [5, 1, 2, 17, 1, 1, 3]}):
        x = torch.cat([xs[i][a:a + take] for i, a, take in entries]).to("cuda", dtype)
        y = part.forward(x, ctx, cache.views()[0]).float().cpu()
        at = 0
        for i, a, take in entries:
            got[i][a:a + take] = y[at:at + take]
            at += take
    for g_, w_ in zip(got, want):
        check(g_, w_, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block(ops, dtype):
    hidden = 64
    norm = NormSpec("rmsnorm", hidden, 1e-5)
    spec = BlockSpec("pre_norm", ShortConvSpec("short_conv", hidden, taps=3, bias=False),
                     SwiGLUSpec("swiglu", hidden, ffn_dim=96,
                                names={"gate": "w1.weight", "up": "w3.weight", "down": "w2.weight"}),
                     {"mixer": (norm, "model.layers.0.operator_norm.weight"),
                      "ffn": (norm, "model.layers.0.ffn_norm.weight")},
                     "model.layers.0.conv.", "model.layers.0.feed_forward.")
    cls = arrangement_class("pre_norm")
    dev, host = tensors_for(cls.params(spec), dtype)
    block = cls(spec, dev, ops, dtype)
    x = torch.randn(23, hidden, generator=torch.Generator().manual_seed(4))
    cfg = {"hidden_size": hidden, "norm_eps": 1e-5, "conv_bias": False}
    want = P.block(x, host, 0, cfg, is_attention=False)
    for cache, ctx, entries in context(ops, mixer_class("short_conv").cache_need(spec.mixer), 8,
                                       [23], {"dtype": dtype, "sizes": [23]}):
        stream = block.forward(Stream(x.cuda(), None), ctx, cache.views()[0])
        out = stream.resid.cpu() + stream.pending.float().cpu()
    check(out, want, dtype)


# ---- parts defined outside the package -----------------------------------------------------

@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    toy.register_toy()
    return write_random_model(str(tmp_path_factory.mktemp("toy")), config_from_dict(toy.TOY), 7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_toy_architecture_on_the_gpu(toy_folder, dtype, schedule):
    model, _ = load_model(toy_folder, dtype, "cuda")
    w = P.read_safetensors(os.path.join(toy_folder, "model.safetensors"))
    rng = random.Random(2)
    reqs = {f"t{i}": [rng.randrange(300) for _ in range(n)] for i, n in enumerate((40, 3, 77, 21, 50))}
    steps = schedules.tail_decode(reqs, 12) if schedule == "tail_decode" else \
        getattr(schedules, schedule)(reqs)
    cache = make_cache(model, 8, schedules.tokens_held(steps, 64) // 8, 4)
    runner = ModelRunner(model, cache, model.ops, use_graphs=False)
    got = schedules.replay(runner, steps)
    b = 1e-5 if dtype == "float32" else 3e-2
    for rid, ids in reqs.items():
        ref = toy.toy_plain_logits(ids, w, toy.TOY)
        for p in range(len(ids)):
            err = float((got[(rid, p)] - ref[p]).abs().max()) / float(ref.abs().max())
            assert err <= b, (rid, p, err)
    assert all(g.pool.in_use == 0 for g in cache.groups)
