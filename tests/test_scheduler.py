"""The scheduler's decisions, without a model: a counting step function stands in for
the runner (the next token is the last token + 1 mod 1000; the idea is the reference's
`CountingBackend`, src/engine.rs:646-696)."""
import pytest
import torch

from rvllm_b200.cache import CacheManager
from rvllm_b200.engine import (Engine, FinishReason, Request, Scheduler, SchedulerConfig, run)
from rvllm_b200.errors import RequestError
from rvllm_b200.parts.base import PagedNeed, StateNeed
from rvllm_b200.sampling import SamplingParams

VOCAB = 1000


class CountingOps:
    def argmax(self, logits):
        return logits.argmax(dim=1).to(torch.int32)


class CountingRunner:
    """Keeps the cache bookkeeping honest (reserve, advance) and records every step."""

    def __init__(self, num_blocks, block_size, slots=64):
        self.cache = CacheManager([PagedNeed(1, 16), StateNeed((2, 4))], [None, None], block_size,
                                  num_blocks, slots, allocate=False)
        self.ops = CountingOps()
        self.device = "cpu"
        self.log = []

    def step(self, entries):
        rows = []
        self.log.append([(e.req, len(e.tokens), self.cache.requests[e.req].computed) for e in entries])
        for e in entries:
            rc = self.cache.requests[e.req]
            total = rc.computed + len(e.tokens)
            assert self.cache.reserve(e.req, total)
            self.cache.advance(e.req, total)
            for w in e.want:
                row = torch.zeros(VOCAB)
                row[(e.tokens[w] + 1) % VOCAB] = 1.0
                rows.append(row)
        self.cache.check()
        return torch.stack(rows) if rows else torch.zeros(0, VOCAB)


def go(requests, num_blocks=64, block_size=4, **cfg):
    runner = CountingRunner(num_blocks, block_size)
    config = SchedulerConfig(block_size=block_size, num_blocks=num_blocks, **cfg)
    result = run(runner, requests, config, context_length=256)
    assert runner.cache.groups[0].pool.in_use == 0 and runner.cache.slots.in_use == 0
    return result, runner


def expected(prompt, n):
    return [(prompt[-1] + 1 + i) % VOCAB for i in range(n)]


def test_outputs_do_not_depend_on_batching():
    reqs = [Request(i, list(range(10 * i, 10 * i + 3 + i)), 6) for i in range(5)]
    together, _ = go(reqs)
    for r in reqs:
        alone, _ = go([r])
        assert together.outputs[r.id] == alone.outputs[r.id] == expected(r.tokens, 6)
    assert all(f == FinishReason.LENGTH for f in together.finish.values())


def test_prompts_are_cut_under_the_token_budget():
    reqs = [Request("a", list(range(50)), 3), Request("b", list(range(100, 130)), 3)]
    result, runner = go(reqs, max_num_batched_tokens=16, prefill_chunk=12)
    assert all(sum(n for _, n, _ in step) <= 16 for step in runner.log)
    assert all(n <= 12 for step in runner.log for _, n, _ in step)
    assert result.outputs["a"] == expected(reqs[0].tokens, 3)
    # portions of one prompt are consecutive and start where the last one ended
    at = 0
    for step in runner.log:
        for rid, n, start in step:
            if rid == "a" and at < 50:
                assert start == at
                at += n
    assert at >= 50


def test_decodes_come_before_portions_and_share_the_step():
    reqs = [Request("short", [1, 2, 3], 8), Request("long", list(range(40)), 2)]
    _, runner = go(reqs, max_num_batched_tokens=12, prefill_chunk=8)
    mixed = [s for s in runner.log if len(s) == 2 and {n == 1 for _, n, _ in s} == {True, False}]
    assert len(mixed) >= 3, "decode tokens and prompt portions should share steps"
    assert all(s[0][1] == 1 for s in mixed)          # the single token is first in the step


def test_arrival_steps_are_respected():
    reqs = [Request("early", [5, 6], 10), Request("late", [7], 2, arrival_step=4)]
    result, runner = go(reqs)
    first_late = next(i for i, s in enumerate(runner.log) if any(r == "late" for r, _, _ in s))
    assert first_late >= 4
    assert result.outputs["late"] == expected([7], 2)


def test_stop_token_finishes_and_is_reported():
    result, _ = go([Request("s", [10], 20, stop_tokens=[14])])
    assert result.outputs["s"] == [11, 12, 13, 14] and result.finish["s"] == FinishReason.STOP


def test_max_running_is_first_come_first_served():
    reqs = [Request(i, [i * 10], 4) for i in range(4)]
    _, runner = go(reqs, max_running=2)
    assert all(len(s) <= 2 for s in runner.log)
    firsts = {}
    for i, s in enumerate(runner.log):
        for rid, _, _ in s:
            firsts.setdefault(rid, i)
    assert firsts[0] <= firsts[1] <= firsts[2] <= firsts[3] and firsts[2] > firsts[0]


def test_when_pages_run_out_the_latest_request_is_preempted_and_recomputed():
    # 12 pages of 4 tokens; three requests that together outgrow them
    reqs = [Request(i, list(range(100 * i, 100 * i + 10)), 14) for i in range(3)]
    result, runner = go(reqs, num_blocks=12, block_size=4)
    assert result.stats.preemptions > 0
    for r in reqs:
        assert result.outputs[r.id] == expected(r.tokens, 14)      # unchanged by preemption
    # a preempted request starts again from position 0 with prompt + generated tokens
    restarts = [(rid, n) for s in runner.log for rid, n, start in s if start == 0]
    assert len(restarts) > len(reqs)
    assert any(n > 10 for rid, n in restarts)


def test_admission_waits_for_pages_instead_of_failing():
    reqs = [Request("a", list(range(30)), 2), Request("b", list(range(30)), 2)]
    result, runner = go(reqs, num_blocks=9, block_size=4)      # 36 tokens: not both at once
    assert result.outputs["a"] == expected(reqs[0].tokens, 2)
    assert result.outputs["b"] == expected(reqs[1].tokens, 2)
    # b gets the one page that a leaves free, then waits until a has finished
    assert runner.log[0] == [("a", 30, 0), ("b", 4, 0)]
    assert all(rid == "a" for rid, _, _ in runner.log[1])
    assert result.stats.preemptions == 0


@pytest.mark.parametrize("req,message", [
    (Request("e", [], 4), "prompt is empty"),
    (Request("z", [1], 0), "max_tokens must be at least 1"),
    (Request("l", list(range(256)), 1), "does not fit the model's 256-token context"),
    (Request("c", list(range(60)), 30), "the pool only holds 64"),
])
def test_requests_that_can_never_run_are_refused(req, message):
    runner = CountingRunner(16, 4)
    s = Scheduler(SchedulerConfig(block_size=4, num_blocks=16), runner.cache, 256)
    with pytest.raises(RequestError, match=message):
        s.add_request(req)


def test_max_tokens_is_clamped_to_the_context():
    result, _ = go([Request("x", list(range(250)), 50)], num_blocks=80)
    assert len(result.outputs["x"]) == 6 and result.finish["x"] == FinishReason.LENGTH


def test_abort_frees_everything():
    runner = CountingRunner(16, 4)
    engine = Engine(runner, SchedulerConfig(block_size=4, num_blocks=16), 256)
    engine.add_request(Request("a", list(range(9)), 50))
    engine.add_request(Request("b", [1], 50, arrival_step=30))
    engine.step(); engine.step()
    assert runner.cache.groups[0].pool.in_use > 0
    engine.abort("a"); engine.abort("b"); engine.abort("nobody")
    assert runner.cache.groups[0].pool.in_use == 0 and not engine.has_work()


def test_seeded_sampling_counts_per_request():
    """The sampler is given, for each row, how many tokens its request has drawn."""
    seen = []

    class Recorder:
        def sample(self, logits, params, counters):
            seen.append(list(counters))
            return logits.argmax(dim=1).tolist()

    runner = CountingRunner(64, 4)
    reqs = [Request("a", [1, 2], 3, sampling=SamplingParams(0.8, 1.0, 5)),
            Request("b", [9], 3, sampling=SamplingParams(0.8, 1.0, 6), arrival_step=1)]
    run(runner, reqs, SchedulerConfig(block_size=4, num_blocks=64), 256, sampler=Recorder())
    assert seen[0] == [0] and [1, 0] in seen and [2, 1] in seen


def test_settled_heap_freezes_and_gives_back(monkeypatch):
    """Inside, what was on the heap is in the permanent generation (the collector's passes skip
    it); afterwards it is back; a heap the caller froze is added to and kept; RVLLM_GC_FREEZE=0
    leaves the collector alone."""
    import gc

    from rvllm_b200.engine import settled_heap
    from rvllm_b200.engine.engine import _FROZEN_AT_IMPORT
    gc.unfreeze()
    assert gc.get_freeze_count() <= _FROZEN_AT_IMPORT
    with settled_heap():
        assert gc.get_freeze_count() > 1000
    assert gc.get_freeze_count() == 0
    gc.freeze()                               # a caller's own freeze is added to and kept
    mine = gc.get_freeze_count()
    assert mine > _FROZEN_AT_IMPORT
    with settled_heap():
        assert gc.get_freeze_count() >= mine
    assert gc.get_freeze_count() >= mine
    gc.unfreeze()
    monkeypatch.setenv("RVLLM_GC_FREEZE", "0")
    with settled_heap():
        assert gc.get_freeze_count() == 0
