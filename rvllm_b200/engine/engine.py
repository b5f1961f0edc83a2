"""The engine loop: scheduler above, step function below, sampler beside.

`Engine.step()` asks the scheduler for a plan, turns it into step entries, runs them
through the runner's one step function, samples the rows that reached the end of their
sequence and reports the tokens back.  `run()` drives a fixed set of requests with
arrival steps to completion, like the reference's `engine::run`
(src/engine.rs:576-637); `Engine` corresponds to its `Engine<B>` (src/engine.rs:216-349)
with the runner in the place of its `Backend` trait (src/engine.rs:29-46).
"""
from __future__ import annotations

import contextlib
import gc
import os
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


@dataclass
class _InFlight:
    """A launched step whose sampled ids have not been read yet."""
    plan: list                      # PlannedEntry list
    ids: object                     # int32 device tensor, one id per sampling entry (or None)
    host: object                    # pinned host copy of `ids` (or None)
    ready: object                   # event recorded after the copy (or None)

    check: object = None            # called with the kernels' status word read beside the ids

    def tokens(self) -> List[int]:
        if self.ids is None:
            return []
        if self.ready is None:
            return self.ids.tolist()
        self.ready.synchronize()
        got = self.host.tolist()
        if self.check is not None:
            # the last word is the kernels' status: a wait that ran out left invalid logits
            self.check(got.pop())
        return got


class Engine:
    """`lookahead`: when every sequence of a launched step is decoding and nothing is waiting,
    the next step is launched, with its tokens fed on the device, *before* the host reads the
    step's sampled ids, so the GPU never waits for the host.  A sequence that turns out to have
    finished (a stop token) has then run one step too many; that step's result for it is
    dropped and its pages were freed only after the launch, in stream order.  The tokens a
    request gets are the same with and without lookahead."""

    def __init__(self, runner, config: SchedulerConfig, context_length: int, sampler=None,
                 lookahead: bool = False):
        self.runner = runner
        self.scheduler = Scheduler(config, runner.cache, context_length)
        self.sampler = sampler or BatchSampler(runner.ops, runner.device)
        self.lookahead = lookahead and hasattr(self.sampler, "sample_device") and \
            hasattr(runner, "is_cuda") and runner.is_cuda
        self._flying: Optional[_InFlight] = None
        self.lookahead_steps = 0

    def add_request(self, req: Request) -> None:
        self.scheduler.add_request(req)

    def abort(self, rid: Hashable) -> None:
        self.scheduler.abort(rid)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ---- launching ---------------------------------------------------------------------

    def _launch(self, plan, device_tokens=None, extra_drawn: int = 0) -> _InFlight:
        """Run a plan's entries and sample on the device; nothing here waits for the GPU.
        `extra_drawn`: tokens every sequence has drawn that are not in `seq.tokens` yet."""
        if device_tokens is None:
            entries = [StepEntry(e.seq.request.id, e.seq.tokens[e.start:e.start + e.count],
                                 (e.count - 1,) if e.samples else ()) for e in plan]
            logits = self.runner.step(entries)
        else:
            entries = [StepEntry(e.seq.request.id, (0,), (0,)) for e in plan]
            logits = self.runner.step(entries, device_tokens=device_tokens)
        who = [e.seq for e in plan if e.samples]
        if not who:
            return _InFlight(plan, None, None, None)
        params = [s.request.sampling for s in who]
        counters = [len(s.generated) + extra_drawn for s in who]
        status = getattr(self.runner.ops, "status_word", None)
        if not self.lookahead:
            ids = self.sampler.sample(logits, params, counters)
            if status is not None:
                self.runner.ops.check_status()
            return _InFlight(plan, _HostIds(ids), None, None)
        import torch
        ids = self.sampler.sample_device(logits, params, counters)
        n = ids.shape[0]
        host = torch.empty(n + (status is not None), dtype=ids.dtype, pin_memory=True)
        host[:n].copy_(ids, non_blocking=True)
        check = None
        if status is not None:
            # the kernels' status word travels with the ids: no extra synchronisation
            word = status(ids.device)
            host[n:].copy_(word, non_blocking=True)
            ops = self.runner.ops
            check = lambda code: ops.raise_for_status(code, ids.device)
        ready = torch.cuda.Event()
        ready.record()
        return _InFlight(plan, ids, host, ready, check)

    def _can_look_ahead(self, plan) -> bool:
        sch = self.scheduler
        if not plan or sch.waiting or len(plan) != len(sch.running):
            return False
        if sch.future and sch.future[0].request.arrival_step <= sch.step_index + 1:
            return False
        for e in plan:
            seq = e.seq
            if not e.samples or e.start + e.count != len(seq.tokens):
                return False
            if len(seq.generated) + 1 >= seq.max_tokens:      # ends by length after this step
                return False
        # pages for one more token each, without preempting anybody
        ps = sch.cfg.block_size
        cache = self.runner.cache
        need = [0] * len(cache.groups)
        for e in plan:
            rc = cache.requests[e.seq.request.id]
            want = -(-(e.start + e.count + 1) // ps)
            for gi, table in enumerate(rc.tables):
                if len(table) < want:
                    need[gi] += want - len(table)
        return all(n <= g.pool.available for n, g in zip(need, cache.groups))

    # ---- one step ----------------------------------------------------------------------

    def step(self) -> List[TokenEvent]:
        flying = self._flying
        self._flying = None
        if flying is None:
            plan = self.scheduler.schedule()
            if not plan:
                return self.scheduler.update(plan, [])
            flying = self._launch(plan)
        nxt = None
        if self.lookahead and flying.ids is not None and self._can_look_ahead(flying.plan):
            from .scheduler import PlannedEntry
            ahead = [PlannedEntry(e.seq, e.start + e.count, 1, True) for e in flying.plan]
            for e in ahead:
                self.runner.cache.reserve(e.seq.request.id, e.start + 1)
            nxt = self._launch(ahead, device_tokens=flying.ids, extra_drawn=1)
            self.lookahead_steps += 1
        events = self.scheduler.update(flying.plan, flying.tokens())
        if nxt is not None:
            # keep only the sequences that are still running; the others ran one step for nothing
            alive = [i for i, e in enumerate(nxt.plan) if e.seq.request.id in self.scheduler.seqs]
            if alive:
                if len(alive) != len(nxt.plan):
                    nxt = _Subset(nxt, alive)
                self._flying = nxt
        return events


class _HostIds:
    """Ids that are already on the host, behind the interface of a device tensor."""

    def __init__(self, ids):
        self._ids = list(ids)

    def tolist(self):
        return self._ids


class _Subset(_InFlight):
    """The rows of a launched step that belong to sequences still running."""

    def __init__(self, base: _InFlight, keep: List[int]):
        import torch
        rows = torch.tensor(keep, dtype=torch.long, device=base.ids.device)
        super().__init__([base.plan[i] for i in keep], base.ids.index_select(0, rows), base.host,
                         base.ready, None)
        self._base, self._keep = base, keep

    def tokens(self) -> List[int]:
        all_tokens = self._base.tokens()
        return [all_tokens[i] for i in self._keep]


_FROZEN_AT_IMPORT = gc.get_freeze_count()


@contextlib.contextmanager
def settled_heap():
    """Keep Python's cyclic garbage collector off what is on the heap already.

    A step with prompt portions is launched kernel by kernel, so a pause of the host is a
    pause of the GPU; the collector's full passes walk every container object of the process
    (the model, the framework's modules: some hundred thousand) and came to a fifth of such
    a workload's time.  On entry garbage is collected once and what remains is moved to the
    permanent generation (`gc.freeze`), which later passes skip; on exit it is moved back.
    Objects made inside are collected as usual.  RVLLM_GC_FREEZE=0 turns it off."""
    if os.environ.get("RVLLM_GC_FREEZE", "1") == "0":
        yield
        return
    # A permanent generation that has grown since this module was imported is somebody else's
    # (a caller who froze their heap): it is added to and then left as it is, because
    # `gc.unfreeze` would thaw their objects too.  (The interpreter itself starts with a few
    # hundred objects there.)
    thaw = gc.get_freeze_count() <= _FROZEN_AT_IMPORT
    gc.collect()
    gc.freeze()
    try:
        yield
    finally:
        if thaw:
            gc.unfreeze()


def run(runner, requests: Sequence[Request], config: SchedulerConfig, context_length: int,
        sampler=None, lookahead: bool = False) -> RunResult:
    """Run `requests` to completion; outputs hold the generated tokens, a stop token
    included when one ended the request."""
    with settled_heap():
        return _run(runner, requests, config, context_length, sampler, lookahead)


def _run(runner, requests, config, context_length, sampler, lookahead) -> RunResult:
    engine = Engine(runner, config, context_length, sampler, lookahead)
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
