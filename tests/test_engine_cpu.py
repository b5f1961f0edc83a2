"""The engine's host side (cache manager, batch packing, step function) driven through
the plain kernel references on the CPU, against the plain whole-sequence model."""
import random

import pytest
import torch

import schedules
from plain_lfm2 import PlainModel
from plain_ops import PlainOps
from rvllm_b200.engine import ModelRunner, load_model, make_cache
from tiny import write_tiny


def _requests(vocab, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.fixture(scope="module", params=["A", "B"])
def setup(request, tmp_path_factory):
    folder = write_tiny(str(tmp_path_factory.mktemp("models")), request.param)
    plain = PlainModel(folder)
    model, cfg = load_model(folder, "float32", "cpu", PlainOps())
    return plain, model, cfg


@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_schedules_match_plain(setup, schedule):
    plain, model, cfg = setup
    reqs = _requests(cfg.vocab_size, [5, 17, 31, 40, 9, 23], seed=3)
    steps = getattr(schedules, schedule)(reqs) if schedule != "tail_decode" else \
        schedules.tail_decode(reqs, tail=6)
    page = 8
    pages = schedules.tokens_held(steps, 64) // page
    cache = make_cache(model, page, pages, 4)
    runner = ModelRunner(model, cache, PlainOps())
    got = schedules.replay(runner, steps)
    assert cache.groups[0].pool.in_use == 0
    for rid, ids in reqs.items():
        ref = plain.logits(ids)
        for p in range(len(ids)):
            assert torch.allclose(got[(rid, p)], ref[p], atol=2e-5, rtol=0), (rid, p)
    if schedule == "mixed":
        # more pages handed out than were ever out at once: some were used again
        assert cache.groups[0].pool.total_allocs > cache.groups[0].pool.high_water
