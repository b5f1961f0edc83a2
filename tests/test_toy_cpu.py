"""Generality of the parts, on the CPU through the plain kernel references: a toy
architecture defined in tests/toy.py (a mixer with its own state, another feed-forward,
another position encoding, a windowed attention group beside a full one, a block that
runs twice, a call that reads another call's cache) is registered, built from a model
folder and stepped under every cut, with no change to the package."""
import os
import random

import pytest
import torch

import schedules
import toy
from plain_lfm2 import read_safetensors
from plain_ops import PlainOps
from rvllm_b200.config import config_from_dict
from rvllm_b200.engine import ModelRunner, load_model, make_cache
from rvllm_b200.weights import write_random_model


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    toy.register_toy()
    folder = write_random_model(str(tmp_path_factory.mktemp("toy")), config_from_dict(toy.TOY), 7)
    model, _ = load_model(folder, "float32", "cpu", PlainOps())
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    return model, w


def test_toy_is_built_from_registered_parts(setup):
    model, _ = setup
    kinds = [type(b.mixer).__name__ for b in model.blocks]
    assert kinds == ["ToyDecay", "Attention", "Attention", "ToyDecay"]
    assert type(model.blocks[0].feed_forward).__name__ == "ScaledRelu"
    assert type(model.blocks[3].feed_forward).__name__ == "SoftRouted"
    needs = model.cache_needs()
    assert needs[5] is None and needs[2] is not None          # the last call owns no cache
    cache = make_cache(model, 4, 64, 4)
    assert len(cache.groups) == 2                              # windowed and full attention
    assert sorted(cache.states) == [0, 4]                      # the two decay calls


@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_toy_under_every_cut(setup, schedule):
    model, w = setup
    rng = random.Random(2)
    reqs = {f"t{i}": [rng.randrange(300) for _ in range(n)] for i, n in enumerate((40, 3, 77, 21, 50))}
    steps = schedules.tail_decode(reqs, 12) if schedule == "tail_decode" else \
        getattr(schedules, schedule)(reqs)
    cache = make_cache(model, 4, schedules.tokens_held(steps, 64) // 4, 4)
    runner = ModelRunner(model, cache, PlainOps())
    got = schedules.replay(runner, steps)
    for rid, ids in reqs.items():
        ref = toy.toy_plain_logits(ids, w, toy.TOY)
        for p in range(len(ids)):
            assert torch.allclose(got[(rid, p)], ref[p], atol=2e-5, rtol=0), (rid, p)
    windowed = next(g for g in cache.groups if g.need.window)
    full = next(g for g in cache.groups if not g.need.window)
    if schedule != "whole":      # a whole prompt reserves all its pages at once
        assert windowed.pool.high_water < full.pool.high_water   # the window gave pages back
    assert all(g.pool.in_use == 0 for g in cache.groups)


def test_a_reused_slot_starts_from_zero(setup):
    """One state slot, two requests one after the other: the second gets the slot the first
    left full of its state, and `ToyDecay` does nothing to clear it.  Its logits are those
    of a fresh sequence because the cache manager clears a slot when it hands it out."""
    model, w = setup
    rng = random.Random(3)
    first = [rng.randrange(300) for _ in range(30)]
    second = [rng.randrange(300) for _ in range(18)]
    cache = make_cache(model, 4, 32, 1)
    runner = ModelRunner(model, cache, PlainOps())
    from rvllm_b200.engine import StepEntry
    runner.add_request("a")
    slot = cache.requests["a"].slot
    runner.step([StepEntry("a", first, ())])
    assert float(cache.states[0][slot].abs().max()) > 0
    runner.end_request("a")
    runner.add_request("b")
    assert cache.requests["b"].slot == slot
    got = runner.step([StepEntry("b", second, range(len(second)))])
    ref = toy.toy_plain_logits(second, w, toy.TOY)
    assert torch.allclose(got.cpu(), ref, atol=2e-5, rtol=0)


def test_post_norms_and_own_distribution(setup):
    model, w = setup
    assert model.blocks[3].post_mixer is not None and model.blocks[3].post_ffn is not None
    assert model.blocks[0].post_mixer is None
    assert "blocks.3.post1.weight" in w and "blocks.0.post1.weight" not in w
    std = float(w["blocks.0.mixer.w.weight"].std())
    assert 0.025 < std < 0.035            # N(0, 0.03) as the part declared, not a named kind


def test_a_place_the_arrangement_does_not_know_is_refused():
    from rvllm_b200.parts import BlockSpec, NormSpec, arrangement_class
    norm = NormSpec("rmsnorm", 8, 1e-5)
    spec = BlockSpec("pre_norm", toy.ToyDecaySpec("toy_decay", 8),
                     toy.ScaledReluSpec("toy_scaled_relu", 8, width=8),
                     {"mixer": (norm, "a"), "ffn": (norm, "b"), "middle": (norm, "c")}, "m.", "f.")
    toy.register_toy()
    with pytest.raises(ValueError, match="no place 'middle'"):
        arrangement_class("pre_norm").params(spec)
