"""Continuous batching: admit requests, cut prompts into portions under a token
budget, decode, finish and free.

A sequence is its prompt plus what it has generated; `computed` says how many of these
tokens are in the cache.  Every step each running sequence brings its next tokens: one
if only the last sampled token is missing (a decode), else a portion of at most
`prefill_chunk` tokens.  Single tokens are scheduled first, then portions in admission
order, then waiting requests first-come-first-served, until `max_num_batched_tokens`
is spent.  A sequence whose portion reaches its last token gets a logits row and
samples its next token.

When pages run out.  Sequences that decode are served first and, if one of them cannot
get the page it needs, the most recently admitted running sequence is preempted: its
pages and state slot are freed, `computed` goes back to 0 and it returns to the front
of the waiting queue; on readmission its prompt *and* the tokens it had generated are
recomputed, after which it continues where it stopped, so its output is unchanged.
A portion that finds no pages simply waits a step.  A request that could never fit the
pool even alone is refused at `add_request`.

The reference's engine admits a request only when its whole prompt fits the free
blocks, prefills it alone, and decodes all running sequences together
(src/engine.rs:351-401, 405-490); its external scheduler crate evicts a sequence when
blocks run out and the engine re-prefills prompt + generated (src/engine.rs:418-433).
Checks at admission and the finish reasons follow src/engine.rs:279-309, 505-539.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..errors import RequestError
from ..sampling.params import GREEDY, SamplingParams


class FinishReason(Enum):
    STOP = "stop"
    LENGTH = "length"


@dataclass
class Request:
    id: Hashable
    tokens: Sequence[int]
    max_tokens: int
    stop_tokens: Sequence[int] = ()
    sampling: SamplingParams = GREEDY
    arrival_step: int = 0


@dataclass
class TokenEvent:
    id: Hashable
    token: int
    finish: Optional[FinishReason] = None
    ttft: Optional[float] = None       # seconds from admission to the first token


@dataclass
class SchedulerConfig:
    block_size: int = 16                   # tokens per page
    num_blocks: int = 0                    # pages in the pool
    max_running: int = 1 << 30             # cap on sequences holding cache
    max_num_batched_tokens: int = 8192     # token budget of a step
    prefill_chunk: Optional[int] = None    # longest prompt portion; None: the budget


@dataclass
class Sequence_:
    request: Request
    tokens: List[int]                      # prompt + generated
    prompt_len: int
    max_tokens: int
    computed: int = 0
    admitted_at: Optional[float] = None
    admission_index: int = -1
    first_token_seen: bool = False
    preemptions: int = 0

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.prompt_len:]

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.computed


@dataclass
class PlannedEntry:
    seq: Sequence_
    start: int
    count: int
    samples: bool                          # the portion reaches the sequence's last token


@dataclass
class SchedulerStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    admitted: int = 0
    finished: int = 0
    max_running: int = 0
    tokens_per_step: List[int] = field(default_factory=list)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache, context_length: int):
        self.cfg = config
        self.cache = cache
        self.context_length = context_length
        self.waiting: Deque[Sequence_] = deque()
        self.future: List[Sequence_] = []        # not yet arrived, by arrival step
        self.running: List[Sequence_] = []       # in admission order
        self.seqs: Dict[Hashable, Sequence_] = {}
        self.step_index = 0
        self._admissions = 0
        self.stats = SchedulerStats()

    # ---- requests --------------------------------------------------------------------

    def add_request(self, req: Request) -> None:
        if req.id in self.seqs:
            raise RequestError(f"request id {req.id!r} is already in use")
        if len(req.tokens) == 0:
            raise RequestError("prompt is empty")
        if req.max_tokens <= 0:
            raise RequestError("max_tokens must be at least 1")
        prompt = len(req.tokens)
        if prompt >= self.context_length:
            raise RequestError(f"prompt is {prompt} tokens, which does not fit the model's "
                               f"{self.context_length}-token context")
        max_tokens = min(req.max_tokens, self.context_length - prompt)
        capacity = self.cfg.num_blocks * self.cfg.block_size
        # the last generated token is never fed back, so it needs no slot
        if prompt + max_tokens - 1 > capacity:
            raise RequestError(f"request needs {prompt + max_tokens - 1} tokens of KV cache "
                               f"but the pool only holds {capacity}")
        seq = Sequence_(req, list(req.tokens), prompt, max_tokens)
        self.seqs[req.id] = seq
        if req.arrival_step <= self.step_index:
            self.waiting.append(seq)
        else:
            self.future.append(seq)
            self.future.sort(key=lambda s: s.request.arrival_step)

    def abort(self, rid: Hashable) -> None:
        seq = self.seqs.pop(rid, None)
        if seq is None:
            return
        if seq in self.running:
            self.running.remove(seq)
            self.cache.free(rid)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        elif seq in self.future:
            self.future.remove(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self.future)

    # ---- one step's plan -------------------------------------------------------------

    def _preempt(self, victim: Sequence_) -> None:
        self.running.remove(victim)
        self.cache.free(victim.request.id)
        victim.computed = 0
        victim.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(victim)

    def schedule(self) -> List[PlannedEntry]:
        while self.future and self.future[0].request.arrival_step <= self.step_index:
            self.waiting.append(self.future.pop(0))
        budget = self.cfg.max_num_batched_tokens
        chunk = self.cfg.prefill_chunk or budget
        plan: List[PlannedEntry] = []

        # 1. sequences that only miss their last sampled token
        for seq in list(self.running):
            if seq not in self.running or seq.pending != 1:
                continue
            if budget < 1:
                break
            rc = self.cache.requests[seq.request.id]
            while rc.tokens <= seq.computed and \
                    not self.cache.can_reserve(seq.request.id, seq.computed + 1):
                victim = self.running[-1]
                if victim is seq and len(self.running) == 1:
                    raise RequestError("a lone sequence cannot get a page: the pool is too "
                                       "small for it")     # add_request rules this out
                self._preempt(victim)
                plan = [e for e in plan if e.seq is not victim]
                if victim is seq:
                    break
            if seq not in self.running:
                continue
            self.cache.reserve(seq.request.id, seq.computed + 1)
            plan.append(PlannedEntry(seq, seq.computed, 1, True))
            budget -= 1

        # 2. portions of running sequences
        for seq in self.running:
            if seq.pending <= 1 or budget < 1:
                continue
            n = min(seq.pending, chunk, budget)
            if n < seq.pending and n < 2 and seq.pending > 1:
                continue                    # do not spend the budget's last token on a sliver
            while n >= 1 and not self.cache.can_reserve(seq.request.id, seq.computed + n):
                n = min(n - 1, self._tokens_that_fit(seq))
            if n < 1:
                continue
            self.cache.reserve(seq.request.id, seq.computed + n)
            plan.append(PlannedEntry(seq, seq.computed, n, seq.computed + n == len(seq.tokens)))
            budget -= n

        # 3. waiting requests, first come first served
        while self.waiting and budget >= 1 and len(self.running) < self.cfg.max_running:
            seq = self.waiting[0]
            if not self.cache.can_add():
                break
            n = min(seq.pending, chunk, budget)
            fit = self._tokens_that_fit(seq, fresh=True)
            n = min(n, fit)
            if n < 1 or (n < seq.pending and n < min(2, seq.pending)):
                break                       # head-of-line blocking, as in the reference
            self.waiting.popleft()
            self.cache.add(seq.request.id)
            self.cache.reserve(seq.request.id, n)
            seq.admission_index = self._admissions
            self._admissions += 1
            if seq.admitted_at is None:
                seq.admitted_at = time.perf_counter()
            self.running.append(seq)
            self.stats.admitted += 1
            plan.append(PlannedEntry(seq, 0, n, n == len(seq.tokens)))
            budget -= n

        if not plan and len(self.running) > 1:
            # every running sequence waits for pages that only another one could free
            self._preempt(self.running[-1])
            return self.schedule()
        self.stats.max_running = max(self.stats.max_running, len(self.running))
        return plan

    def _tokens_that_fit(self, seq: Sequence_, fresh: bool = False) -> int:
        """How many more tokens of `seq` the free pages can take."""
        ps = self.cfg.block_size
        free_pages = min(g.pool.available for g in self.cache.groups) if self.cache.groups \
            else 1 << 30
        have = 0 if fresh else self.cache.requests[seq.request.id].tokens
        reserved_pages = -(-have // ps)
        room = (reserved_pages + free_pages) * ps - seq.computed
        return max(0, room)

    # ---- after the step --------------------------------------------------------------

    def update(self, plan: List[PlannedEntry], sampled: Sequence[int]) -> List[TokenEvent]:
        """`sampled` holds one token per planned entry with `samples` set, in plan order."""
        events: List[TokenEvent] = []
        k = 0
        total = 0
        for e in plan:
            seq = e.seq
            if self.seqs.get(seq.request.id) is not seq:      # aborted while the step ran
                k += int(e.samples)
                continue
            seq.computed = e.start + e.count
            total += e.count
            if e.count == 1 and e.start >= seq.prompt_len:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += e.count
            if not e.samples:
                continue
            token = int(sampled[k])
            k += 1
            seq.tokens.append(token)
            finish = None
            if token in seq.request.stop_tokens:
                finish = FinishReason.STOP
            elif len(seq.generated) >= seq.max_tokens:
                finish = FinishReason.LENGTH
            ttft = None
            if not seq.first_token_seen:
                seq.first_token_seen = True
                ttft = time.perf_counter() - seq.admitted_at
            events.append(TokenEvent(seq.request.id, token, finish, ttft))
            if finish is not None:
                self.running.remove(seq)
                self.cache.free(seq.request.id)
                del self.seqs[seq.request.id]
                self.stats.finished += 1
        self.stats.steps += 1
        self.stats.tokens_per_step.append(total)
        self.step_index += 1
        return events
