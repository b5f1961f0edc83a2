"""The engine loop: scheduler above, step function below, sampler beside.

`Engine.step()` asks the scheduler for a plan, turns it into step entries, runs them
through the runner's one step function, samples the rows that reached the end of their
sequence and reports the tokens back.  `run()` drives a fixed set of requests with
arrival steps to completion, like the reference's `engine::run`
(src/engine.rs:576-637); `Engine` corresponds to its `Engine<B>` (src/engine.rs:216-349)
with the runner in the place of its `Backend` trait (src/engine.rs:29-46).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from ..sampling.sampler import BatchSampler
from .batch import StepEntry
from .scheduler import FinishReason, Request, Scheduler, SchedulerConfig, TokenEvent


@dataclass
class RunStats:
    steps: int = 0
    elapsed: float = 0.0
    output_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    page_allocs: int = 0
    pages_high_water: int = 0
    ttft: Dict[Hashable, float] = field(default_factory=dict)


@dataclass
class RunResult:
    outputs: Dict[Hashable, List[int]]
    finish: Dict[Hashable, FinishReason]
    stats: RunStats


class Engine:
    def __init__(self, runner, config: SchedulerConfig, context_length: int, sampler=None):
        self.runner = runner
        self.scheduler = Scheduler(config, runner.cache, context_length)
        self.sampler = sampler or BatchSampler(runner.ops, runner.device)

    def add_request(self, req: Request) -> None:
        self.scheduler.add_request(req)

    def abort(self, rid: Hashable) -> None:
        self.scheduler.abort(rid)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> List[TokenEvent]:
        plan = self.scheduler.schedule()
        entries = [StepEntry(e.seq.request.id, e.seq.tokens[e.start:e.start + e.count],
                             (e.count - 1,) if e.samples else ()) for e in plan]
        sampled: List[int] = []
        if entries:
            logits = self.runner.step(entries)
            who = [e.seq for e in plan if e.samples]
            sampled = self.sampler.sample(logits, [s.request.sampling for s in who],
                                          [len(s.generated) for s in who])
        return self.scheduler.update(plan, sampled)


def run(runner, requests: Sequence[Request], config: SchedulerConfig, context_length: int,
        sampler=None) -> RunResult:
    """Run `requests` to completion; outputs hold the generated tokens, a stop token
    included when one ended the request."""
    engine = Engine(runner, config, context_length, sampler)
    for r in requests:
        engine.add_request(r)
    outputs: Dict[Hashable, List[int]] = {r.id: [] for r in requests}
    finish: Dict[Hashable, FinishReason] = {}
    stats = RunStats()
    t0 = time.perf_counter()
    while engine.has_work():
        for ev in engine.step():
            outputs[ev.id].append(ev.token)
            if ev.ttft is not None:
                stats.ttft[ev.id] = ev.ttft
            if ev.finish is not None:
                finish[ev.id] = ev.finish
    stats.elapsed = time.perf_counter() - t0
    s = engine.scheduler.stats
    stats.steps, stats.prefill_tokens, stats.decode_tokens = s.steps, s.prefill_tokens, s.decode_tokens
    stats.preemptions = s.preemptions
    stats.output_tokens = sum(len(v) for v in outputs.values())
    if runner.cache.groups:
        stats.page_allocs = sum(g.pool.total_allocs for g in runner.cache.groups)
        stats.pages_high_water = max(g.pool.high_water for g in runner.cache.groups)
    return RunResult(outputs, finish, stats)
