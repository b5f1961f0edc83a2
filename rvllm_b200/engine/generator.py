"""The Python entry point, in the manner of the reference's `Generator`
(src/generator.rs:97-196):

    gen = Generator.load(model_dir)                     # device "cuda", dtype "bfloat16"
    text = gen.complete("prompt", GenerateOptions(max_tokens=64))
    ids  = gen.complete([5, 17, 3], GenerateOptions(max_tokens=8))   # token ids in and out

`GenerateOptions` keeps the reference's fields and defaults (max_tokens 64, greedy,
block_size 16, src/generator.rs:24-36) and adds the pool and scheduling knobs of the
command line.  Text prompts need a `tokenizer.json` beside the model and the
`tokenizers` package; token-id prompts need neither.  As in the reference, the pool
holds enough pages for every request's prompt + max_tokens unless `num_blocks` says
otherwise (src/generator.rs:152-157), and a trailing stop token is stripped from the
result (src/generator.rs:173-182).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import torch

from ..sampling.params import SamplingParams
from .engine import RunResult, run
from .loading import load_model, make_cache
from .runner import ModelRunner
from .scheduler import Request, SchedulerConfig


def graphs_default() -> bool:
    """Single-token steps replay a captured CUDA graph unless RVLLM_NO_GRAPHS=1."""
    return os.environ.get("RVLLM_NO_GRAPHS", "0") != "1"


@dataclass
class GenerateOptions:
    max_tokens: int = 64
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    block_size: int = 16
    num_blocks: Optional[int] = None          # default: room for every request
    prefill_chunk: Optional[int] = None       # longest prompt portion per step
    max_batched_tokens: int = 8192            # token budget of a step
    max_running: Optional[int] = None
    stop_tokens: Optional[Sequence[int]] = None   # default: the model's eos token

    @property
    def sampling(self) -> SamplingParams:
        return SamplingParams(self.temperature, self.top_p, self.seed)


Prompt = Union[str, Sequence[int]]


class Generator:
    def __init__(self, model, config, tokenizer=None):
        self.model = model
        self.config = config
        self.ops = model.ops
        self.tokenizer = tokenizer
        self._runner = None
        self._runner_key = None
        self.last_result: Optional[RunResult] = None
        # launch the next decode step before reading the current one's tokens
        self.lookahead = os.environ.get("RVLLM_LOOKAHEAD", "1") != "0"

    @classmethod
    def load(cls, model_dir: str, tokenizer: Optional[str] = None, device: str = "cuda",
             dtype: str = "bfloat16") -> "Generator":
        model, config = load_model(model_dir, dtype, device)
        tok_path = tokenizer or os.path.join(model_dir, "tokenizer.json")
        tok = None
        if os.path.isfile(tok_path):
            try:
                from tokenizers import Tokenizer
                tok = Tokenizer.from_file(tok_path)
            except ImportError:
                tok = None
        return cls(model, config, tok)

    # ---- helpers ---------------------------------------------------------------------

    def _encode(self, prompt: Prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs tokenizer.json beside the model (and the "
                                 "tokenizers package); pass token ids instead")
            return list(self.tokenizer.encode(prompt).ids)
        return [int(t) for t in prompt]

    def _runner_for(self, block_size: int, num_blocks: int, slots: int,
                    exact: bool = True) -> ModelRunner:
        """The runner with a pool of `num_blocks` pages and `slots` state slots.  `exact`
        False (the pool was sized for this call's requests, not asked for by the caller): a
        runner from an earlier call whose pool is at least as large is used again, with its
        captured launch sequences, instead of a new pool and new captures for every call."""
        if not exact:
            slots = max(slots, 8)             # state slots are small; fewer rebuilds for small batches
        have = self._runner
        if have is not None and not exact and self._runner_key[0] == block_size \
                and have.cache.num_pages >= num_blocks and have.cache.max_requests >= slots:
            return have
        key = (block_size, num_blocks, slots)
        if self._runner_key != key:
            if not exact and have is not None and self._runner_key[0] == block_size:
                # grow by half at least, so that calls of slowly growing size do not each rebuild
                num_blocks = max(num_blocks, have.cache.num_pages + have.cache.num_pages // 2)
                slots = max(slots, have.cache.max_requests)
                key = (block_size, num_blocks, slots)
            self._runner = have = None
            cache = make_cache(self.model, block_size, num_blocks, slots)
            self._runner = ModelRunner(self.model, cache, self.ops, use_graphs=graphs_default())
            self._runner_key = key
        return self._runner

    # ---- the calls -------------------------------------------------------------------

    def complete(self, prompt: Prompt, opts: Optional[GenerateOptions] = None):
        return self.complete_batch([prompt], opts)[0]

    def complete_batch(self, prompts: Sequence[Prompt], opts: Optional[GenerateOptions] = None,
                       arrival_steps: Optional[Sequence[int]] = None):
        opts = opts or GenerateOptions()
        ids = [self._encode(p) for p in prompts]
        result = self.generate_ids(ids, opts, arrival_steps)
        stops = set(self._stop_tokens(opts))
        outs = []
        for i, p in enumerate(prompts):
            toks = list(result.outputs[i])
            if toks and toks[-1] in stops:
                toks.pop()
            outs.append(self.tokenizer.decode(toks) if isinstance(p, str) else toks)
        return outs

    def _stop_tokens(self, opts: GenerateOptions) -> List[int]:
        if opts.stop_tokens is not None:
            return list(opts.stop_tokens)
        eos = self.model.spec.eos_token_id
        return [] if eos is None else [eos]

    def generate_ids(self, prompts: Sequence[Sequence[int]], opts: GenerateOptions,
                     arrival_steps: Optional[Sequence[int]] = None) -> RunResult:
        """Run token-id prompts to completion; request i has id i."""
        context = self.model.spec.max_position
        bs = opts.block_size
        if opts.num_blocks is not None:
            num_blocks = opts.num_blocks
        else:
            num_blocks = sum(max(1, -(-min(len(p) + opts.max_tokens, context) // bs))
                             for p in prompts)
        slots = min(len(prompts), opts.max_running) if opts.max_running else len(prompts)
        runner = self._runner_for(bs, num_blocks, max(1, slots), exact=opts.num_blocks is not None)
        num_blocks = runner.cache.num_pages
        for rid in list(runner.cache.requests):       # left behind by a call that raised
            runner.end_request(rid)
        cfg = SchedulerConfig(block_size=bs, num_blocks=num_blocks,
                              max_running=opts.max_running or (1 << 30),
                              max_num_batched_tokens=opts.max_batched_tokens,
                              prefill_chunk=opts.prefill_chunk)
        stops = self._stop_tokens(opts)
        requests = []
        for i, p in enumerate(prompts):
            arrival = arrival_steps[i] if arrival_steps and i < len(arrival_steps) else 0
            vocab = self.model.spec.vocab_size
            if any(t < 0 or t >= vocab for t in p):
                raise ValueError(f"prompt {i} has a token id outside the vocabulary of {vocab}")
            requests.append(Request(i, list(p), opts.max_tokens, stops,
                                    SamplingParams(opts.temperature, opts.top_p, opts.seed + i),
                                    arrival))
        self.last_result = run(runner, requests, cfg, context, lookahead=self.lookahead)
        return self.last_result
