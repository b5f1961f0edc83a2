"""The step function: run a batch of (request, its next tokens) from the cache and
return the logits at the wanted places.

`ModelRunner.step` is the only way tokens reach the model: generation, the command
line, the Python entry point and trace replay all call it.  It reserves pages for
the new tokens, packs the batch, runs the model once over exactly the tokens it was
given, and marks them written.  A step made only of single tokens runs as a replayed
CUDA graph when graphs are enabled (one launch instead of some hundred).

The reference has two forward shapes instead (one whole prompt alone, or N single
tokens, src/engine.rs:351-401, 405-490) behind `Backend::forward_sample`
(src/engine.rs:29-46).
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import gc
import os
import weakref

import torch

from ..errors import CacheError
from .batch import BatchBuilder, StepContext, StepEntry


class ModelRunner:
    def __init__(self, model, cache, ops, use_graphs: bool = False):
        self.model = model
        self.cache = cache
        self.ops = ops
        self.device = model.device
        self.is_cuda = torch.device(self.device).type == "cuda"
        self.builder = BatchBuilder(cache, ops, self.device, pinned=self.is_cuda)
        self.use_graphs = use_graphs and self.is_cuda
        self._graphs: Dict[Tuple[int, int], "_DecodeGraph"] = {}
        self._shape_graphs: Dict[tuple, "_ShapeGraph"] = {}
        self._seen_shapes = set()
        self.max_shape_graphs = 16
        self._mixed_graphs: Dict[tuple, "_MixedGraph"] = {}
        self.max_mixed_graphs = int(os.environ.get("RVLLM_MIXED_GRAPHS", "32"))
        self.mixed_graph_idle_steps = 1024
        self.steps = 0
        self.graph_steps = 0
        self.captures = 0                # launch sequences captured so far
        self._graph_pool = None
        self.capture_failures = 0
        self._reserve_workspace()

    def _reserve_workspace(self) -> None:
        """Size the kernels' shared scratch for the largest step this cache allows (padded
        as replayed steps pad: request count and block-table width to powers of two), so
        that it never has to be replaced while a captured launch sequence names it."""
        reserve = getattr(self.ops, "reserve_scratch", None)
        if reserve is None or not self.is_cuda:
            return
        from ..parts.base import mixer_class
        cache, spec = self.cache, self.model.spec
        ps = cache.page_size
        tokens = min(spec.max_position, max(1, cache.num_pages) * ps)
        blocks = -(-tokens // ps)
        context = max(16, 1 << (blocks - 1).bit_length()) * ps
        requests = 1 << (max(1, cache.max_requests) - 1).bit_length()
        need = 0
        for call in spec.order:
            m = spec.layers[call.layer].mixer
            need = max(need, mixer_class(m.kind).workspace_bytes(m, self.ops, requests, context))
        reserve(need, self.device)

    def graph_pool(self):
        """The memory pool that this runner's captured launch sequences share."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    # ---- requests ----------------------------------------------------------------

    def add_request(self, req: Hashable) -> None:
        self.cache.add(req)

    def end_request(self, req: Hashable) -> None:
        self.cache.free(req)

    def computed(self, req: Hashable) -> int:
        return self.cache.requests[req].computed

    # ---- the step ----------------------------------------------------------------

    def step(self, entries: Sequence[StepEntry], device_tokens=None) -> torch.Tensor:
        """float32 logits [wanted, vocab], in the order of the entries and of `want`.
        With `device_tokens` (int32 device tensor, one id per entry) every entry brings one
        token whose id is taken from that tensor instead of `entry.tokens`."""
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32,
                               device=self.device)
        requests, limit = self.cache.requests, self.model.spec.max_position
        if len({e.req for e in entries}) != len(entries):
            raise ValueError("a request appears twice in one step")
        totals = []
        for e in entries:
            rc = requests.get(e.req)
            if rc is None:
                raise CacheError(f"request {e.req!r} is not live")
            total = rc.computed + len(e.tokens)
            if total > limit:
                raise ValueError(f"request {e.req!r}: {total} tokens exceed the model's "
                                 f"{limit} positions")
            totals.append(total)
        for e, total in zip(entries, totals):
            if total > requests[e.req].tokens and not self.cache.reserve(e.req, total):
                raise CacheError(f"out of pages: request {e.req!r} needs room for "
                                 f"{total} tokens")
        # single tokens first; logits keep the callers' order through logit_rows
        order = sorted(range(len(entries)), key=lambda i: len(entries[i].tokens) != 1)
        ordered = [entries[i] for i in order]
        if device_tokens is not None:
            if any(len(e.tokens) != 1 for e in entries):
                raise ValueError("device-fed tokens are for single-token entries only")
            logits = self._run(ordered, device_tokens)
        elif order != list(range(len(entries))):
            # the wanted rows come out in the callers' order: the row list is written that way
            where = {oi: k for k, oi in enumerate(order)}
            logits = self._run(ordered, row_order=[where[i] for i in range(len(entries))])
        else:
            logits = self._run(ordered)
        for e, total in zip(entries, totals):
            self.cache.advance(e.req, total)
        self.steps += 1
        return logits

    def _run(self, ordered: List[StepEntry], device_tokens=None, row_order=None) -> torch.Tensor:
        if self.use_graphs and all(len(e.tokens) == 1 for e in ordered):
            return self._run_graph(ordered, device_tokens)
        if self.use_graphs and device_tokens is None:
            logits = self._run_padded_mixture(ordered, row_order)
            if logits is None:
                logits = self._run_repeated_shape(ordered, row_order)
            if logits is not None:
                return logits
        ctx = self.builder.build(ordered, row_order=row_order)
        if device_tokens is not None:
            ctx.token_ids[:len(ordered)].copy_(device_tokens)
        return self.model.forward(ctx, self.cache.views())

    def _run_padded_mixture(self, ordered: List[StepEntry], row_order=None) -> Optional[torch.Tensor]:
        """Steps with prompt portions, padded to sizes that come again: D single-token
        requests (a power of two), P prompt portions (a power of two, one more than there
        are), T tokens in all (a multiple of 64, of 128 above 1,024, of 256 above 4,096) and a
        block-table width as in single-token steps.  The second step that pads to the same
        sizes is captured, and every later one replayed, whatever the portions' lengths and
        the requests are: in live traffic exact shapes hardly ever come twice, and a step of
        a small model launched kernel by kernel waits for the host (about 1.8 ms for some 140
        launches).  Returns None when this step has to go another way."""
        if self.max_mixed_graphs < 0:             # off; 0: the padded layout without captures
            return None
        n_decode = 0
        while n_decode < len(ordered) and len(ordered[n_decode].tokens) == 1:
            n_decode += 1
        n_prefill = len(ordered) - n_decode
        D = 0 if n_decode == 0 else 1 << (n_decode - 1).bit_length()
        P = 1 << n_prefill.bit_length()                  # a power of two above n_prefill
        tokens = D + sum(len(e.tokens) for e in ordered[n_decode:])
        gran = 64 if tokens <= 1024 else (128 if tokens <= 4096 else 256)
        T = -(-tokens // gran) * gran
        W = D + P
        if sum(len(e.want) for e in ordered) > W:
            return None
        ps = self.cache.page_size
        ctx_max = max(self.cache.requests[e.req].computed + len(e.tokens) for e in ordered)
        blocks = -(-ctx_max // ps)
        block_bucket = max(16, 1 << (blocks - 1).bit_length())
        key = (D, P, T, block_bucket)
        g = self._mixed_graphs.get(key)
        if g is None:
            seen = ("mixed",) + key
            first_time = seen not in self._seen_shapes
            if first_time:
                if len(self._seen_shapes) > 4096:
                    self._seen_shapes.clear()
                self._seen_shapes.add(seen)
            if first_time or self.max_mixed_graphs == 0:
                return self._padded_eagerly(ordered, row_order, key)
            if len(self._mixed_graphs) >= self.max_mixed_graphs:
                # room for the sizes that come now, if a launch sequence has not been replayed
                # for a long time (capturing costs several steps' time: sizes that take turns
                # must not push one another out); nothing of it may still be running when its
                # memory goes
                oldest = min(self._mixed_graphs, key=lambda k: self._mixed_graphs[k].last_used)
                if self.steps - self._mixed_graphs[oldest].last_used < self.mixed_graph_idle_steps:
                    return self._padded_eagerly(ordered, row_order, key)
                torch.cuda.synchronize()
                del self._mixed_graphs[oldest]
                self._seen_shapes.discard(("mixed",) + oldest)
            g = _MixedGraph(self, key)
            self._mixed_graphs[key] = g
        if g.broken:
            return self._padded_eagerly(ordered, row_order, key)
        g.last_used = self.steps
        try:
            logits = g.run(ordered, row_order)
        except RuntimeError as e:
            if g.graph is not None and not g.capturing:
                raise
            g.broken = True
            g.graph = None
            self.capture_failures += 1
            import warnings
            warnings.warn(f"capturing a graph for steps padded to {T} tokens failed ({e}); "
                          f"running such steps without it")
            return None
        self.graph_steps += 1
        return logits

    def _padded_eagerly(self, ordered, row_order, key) -> torch.Tensor:
        """The step in the padded layout, launched kernel by kernel: the same kernels on the
        same sizes as the replayed launch sequence of these sizes, so a position's logits do
        not depend on whether its step had been captured yet."""
        D, P, T, block_bucket = key
        ctx = self.builder.build(ordered, pad_blocks=block_bucket, row_order=row_order,
                                 pad_mixed=(D, P, T, D + P))
        ctx.max_ctx_len = block_bucket * self.cache.page_size
        ctx.max_q_len = max(1, T - D)
        return self.model.forward(ctx, self.cache.views())[:ctx.n_wanted]

    def _run_repeated_shape(self, ordered: List[StepEntry], row_order=None) -> Optional[torch.Tensor]:
        """Steps with prompt portions: the second time the same shape comes (the same token
        counts, wanted places and block-table width, as with a fixed portion size), its launch
        sequence is captured, and from then on replayed.  Returns None when this step has to
        be launched kernel by kernel."""
        ps = self.cache.page_size
        ctx_max = max(self.cache.requests[e.req].computed + len(e.tokens) for e in ordered)
        blocks = -(-ctx_max // ps)
        block_bucket = max(16, 1 << (blocks - 1).bit_length())
        key = (tuple(len(e.tokens) for e in ordered), tuple(tuple(e.want) for e in ordered),
               block_bucket, tuple(row_order) if row_order is not None else None)
        g = self._shape_graphs.get(key)
        if g is None:
            if key not in self._seen_shapes:
                if len(self._seen_shapes) > 4096:
                    self._seen_shapes.clear()
                self._seen_shapes.add(key)
                return None
            if len(self._shape_graphs) >= self.max_shape_graphs:
                return None
            g = _ShapeGraph(self, key, block_bucket)
            self._shape_graphs[key] = g
        if g.broken:
            return None
        try:
            logits = g.run(ordered, row_order)
        except RuntimeError as e:
            if g.graph is not None and not g.capturing:
                raise
            g.broken = True
            g.graph = None
            self.capture_failures += 1
            import warnings
            warnings.warn(f"capturing a graph for a step of {sum(key[0])} tokens failed ({e}); "
                          f"running such steps without a graph")
            return None
        self.graph_steps += 1
        return logits

    def decode_greedy(self, reqs: Sequence[Hashable], first_tokens: Sequence[int],
                      steps: int) -> torch.Tensor:
        """`steps` greedy single-token steps for live requests `reqs` with no host round
        trip: the argmax of one step is the next step's token, on the device.  Returns
        the sampled ids, int32 [steps, len(reqs)], on the device.  The first row are the
        successors of `first_tokens`."""
        r = len(reqs)
        prev = torch.tensor(list(first_tokens), dtype=torch.int32, device=self.device)
        out = torch.empty((steps, r), dtype=torch.int32, device=self.device)
        for k in range(steps):
            entries = [StepEntry(q, (0,), (0,)) for q in reqs]
            for e in entries:
                total = self.cache.requests[e.req].computed + 1
                if total > self.model.spec.max_position:
                    raise ValueError(f"request {e.req!r}: {total} tokens exceed the model's "
                                     f"{self.model.spec.max_position} positions")
                if not self.cache.reserve(e.req, total):
                    raise CacheError(f"out of pages: request {e.req!r} needs room for "
                                     f"{total} tokens")
            logits = self._run(entries, device_tokens=prev)
            prev = self.ops.argmax(logits[:r])
            out[k].copy_(prev)
            for e in entries:
                self.cache.advance(e.req, self.cache.requests[e.req].computed + 1)
            self.steps += 1
        return out

    # ---- replayed single-token steps ---------------------------------------------------

    def _run_graph(self, ordered: List[StepEntry], device_tokens=None) -> torch.Tensor:
        ps = self.cache.page_size
        r = len(ordered)
        bucket = 1 << (r - 1).bit_length()
        ctx_max = max(self.cache.requests[e.req].computed + 1 for e in ordered)
        blocks = -(-ctx_max // ps)
        block_bucket = max(16, 1 << (blocks - 1).bit_length())
        # every row's logits are produced inside the graph; the wanted ones are picked after
        full = ordered
        key = (bucket, block_bucket)
        g = self._graphs.get(key)
        if g is None:
            g = _DecodeGraph(self, bucket, block_bucket)
            self._graphs[key] = g
        logits = None
        if not g.broken:
            try:
                logits = g.run(full, device_tokens)
            except RuntimeError as e:
                if g.graph is not None and not g.capturing:
                    raise                     # a replay failed: not something to hide
                # The capture itself failed (a library call that cannot be captured, for
                # instance).  Nothing has run on real tokens yet, so this step and later ones
                # of this shape are launched kernel by kernel instead.
                g.broken = True
                g.graph = None
                self.capture_failures += 1
                import warnings
                warnings.warn(f"capturing a decode graph for batch {bucket} failed ({e}); "
                              f"running such steps without a graph")
        if logits is None:
            ctx = self.builder.build(ordered)
            if device_tokens is not None:
                ctx.token_ids[:r].copy_(device_tokens)
            return self.model.forward(ctx, self.cache.views())
        self.graph_steps += 1
        rows = [i for i, e in enumerate(ordered) for _ in e.want]
        if rows == list(range(r)):
            return logits[:r]
        return logits[torch.tensor(rows, device=logits.device, dtype=torch.long)]


def _capture(graph, fn, pool=None):
    """Capture `fn` into `graph`.  Python's cyclic garbage collector must not run meanwhile:
    if it destroyed an older graph or freed device memory during the capture, the capture
    would be invalidated (and a graph destroyed from a destructor aborts the process), so
    garbage is collected before and collection is off during the capture."""
    torch.cuda.synchronize()
    gc.collect()
    # A matrix-library workspace cached from a capture whose memory pool is gone would be
    # used again on the capture stream: drop the cached workspaces first.
    clear = getattr(torch._C, "_cuda_clearCublasWorkspaces", None)
    if clear is not None:
        clear()
    was_enabled = gc.isenabled()
    gc.disable()
    # `torch.cuda.graph` would also give every cached block back to the driver first
    # (`empty_cache`), after which the steps that follow pay for fresh allocations, by
    # milliseconds and not the same every time: the capture is begun and ended by hand
    global _capture_stream
    if _capture_stream is None:
        _capture_stream = torch.cuda.Stream()
    _capture_stream.wait_stream(torch.cuda.current_stream())
    try:
        with torch.cuda.stream(_capture_stream):
            # one memory pool for all of a runner's graphs: a later capture finds the blocks of
            # an earlier one's dead intermediates instead of asking the driver for new ones
            # (outputs that a graph object still holds are live and are not handed out again)
            if pool is not None:
                graph.capture_begin(pool=pool)
            else:
                graph.capture_begin()
            try:
                out = fn()
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(_capture_stream)
        return out
    finally:
        if was_enabled:
            gc.enable()


_capture_stream = None


class _DecodeGraph:
    """A captured launch sequence for `bucket` single-token requests whose block tables
    are `block_bucket` wide.  Its index arrays live at fixed addresses; a step refills
    them and replays."""

    def __init__(self, runner: ModelRunner, bucket: int, block_bucket: int):
        self.runner = weakref.proxy(runner)     # no cycle: graphs die with their runner
        self.bucket = bucket
        self.block_bucket = block_bucket
        n_groups = len(runner.cache.groups)
        words = 16 * bucket + 64 + n_groups * (bucket * (block_bucket + 1) + 8)
        self.host = torch.empty(words, dtype=torch.int32, pin_memory=True)
        self.dev = torch.empty(words, dtype=torch.int32, device=runner.device)
        self.graph = None
        self.logits = None
        self.broken = False
        self.capturing = False

    def _build(self, entries) -> StepContext:
        ctx = self.runner.builder.build(entries, pad_reqs=self.bucket,
                                        pad_blocks=self.block_bucket,
                                        buffers=(self.host, self.dev))
        # launch sizes that depend on the context length must cover every later replay
        ctx.max_ctx_len = self.block_bucket * self.runner.cache.page_size
        return ctx

    def run(self, entries, device_tokens=None) -> torch.Tensor:
        model, views = self.runner.model, self.runner.cache.views()
        if self.graph is None:
            # An eager run over padding only comes first: it initialises the matrix
            # library for these shapes outside the capture and, being all padding,
            # writes to no cache (a second run of real tokens would shift the
            # convolution states twice).
            warm = self._build([])
            model.forward(warm, views)
            torch.cuda.synchronize()
            ctx = self._build(entries)
            if device_tokens is not None:
                ctx.token_ids[:len(entries)].copy_(device_tokens)
            launches = model.ops.launches
            graph = torch.cuda.CUDAGraph()
            self.capturing = True
            try:
                self.logits = _capture(graph, lambda: model.forward(ctx, views), self.runner.graph_pool())
            finally:
                self.capturing = False
            self.graph = graph
            self.runner.captures += 1
            self.kernels_per_replay = model.ops.launches - launches
        else:
            ctx = self._build(entries)
            if device_tokens is not None:
                ctx.token_ids[:len(entries)].copy_(device_tokens)
        self.graph.replay()
        model.ops.launches += self.kernels_per_replay
        return self.logits


class _MixedGraph:
    """A captured launch sequence for steps of any mixture padded to (D single-token requests,
    P prompt portions, T tokens, block tables `block_bucket` wide): `BatchBuilder.build` with
    `pad_mixed`.  Its index arrays live at fixed addresses; a step refills them and replays.
    Launch sizes that depend on a portion's length or a context's are taken from the padded
    sizes, so that they cover every later replay."""

    def __init__(self, runner: ModelRunner, key):
        self.runner = weakref.proxy(runner)     # no cycle: graphs die with their runner
        self.D, self.P, self.T, self.block_bucket = key
        self.last_used = 0
        R, W = self.D + self.P, self.D + self.P
        n_groups = len(runner.cache.groups)
        words = 4 * self.T + 8 * R + W + 64 + n_groups * (self.T + R * self.block_bucket + 8)
        self.host = torch.empty(words, dtype=torch.int32, pin_memory=True)
        self.dev = torch.empty(words, dtype=torch.int32, device=runner.device)
        self.graph = None
        self.logits = None
        self.broken = False
        self.capturing = False
        self.kernels_per_replay = 0

    def _build(self, entries, row_order=None) -> StepContext:
        runner = self.runner
        ctx = runner.builder.build(entries, pad_blocks=self.block_bucket,
                                   buffers=(self.host, self.dev), row_order=row_order,
                                   pad_mixed=(self.D, self.P, self.T, self.D + self.P))
        ctx.max_ctx_len = self.block_bucket * runner.cache.page_size
        ctx.max_q_len = max(1, self.T - self.D)
        return ctx

    def run(self, entries, row_order=None) -> torch.Tensor:
        model, views = self.runner.model, self.runner.cache.views()
        if self.graph is None:
            # no warm-up run: a step of these padded sizes has already run once, kernel by
            # kernel (`_padded_eagerly`), so the matrix library has met the shapes
            ctx = self._build(entries, row_order)
            launches = model.ops.launches
            graph = torch.cuda.CUDAGraph()
            self.capturing = True
            try:
                self.logits = _capture(graph, lambda: model.forward(ctx, views), self.runner.graph_pool())
            finally:
                self.capturing = False
            self.graph = graph
            self.runner.captures += 1
            self.kernels_per_replay = model.ops.launches - launches
        else:
            ctx = self._build(entries, row_order)
        self.graph.replay()
        model.ops.launches += self.kernels_per_replay
        return self.logits[:ctx.n_wanted]


class _ShapeGraph:
    """A captured launch sequence for one exact step shape (token counts, wanted places,
    block-table width).  It is captured when the shape comes for the second time, so the
    libraries have already run these sizes once outside a capture and no warm-up run is
    needed (a warm-up on real tokens would apply the cache updates twice)."""

    def __init__(self, runner: ModelRunner, key, block_bucket: int):
        self.runner = weakref.proxy(runner)     # no cycle: graphs die with their runner
        self.block_bucket = block_bucket
        n_tokens, n_reqs = sum(key[0]), len(key[0])
        n_want = sum(len(w) for w in key[1])
        n_groups = len(runner.cache.groups)
        words = 4 * n_tokens + 8 * n_reqs + n_want + 64 + \
            n_groups * (n_tokens + n_reqs * block_bucket + 8)
        self.host = torch.empty(words, dtype=torch.int32, pin_memory=True)
        self.dev = torch.empty(words, dtype=torch.int32, device=runner.device)
        self.graph = None
        self.logits = None
        self.broken = False
        self.capturing = False
        self.kernels_per_replay = 0

    def run(self, entries, row_order=None) -> torch.Tensor:
        runner = self.runner
        ctx = runner.builder.build(entries, pad_blocks=self.block_bucket,
                                   buffers=(self.host, self.dev), row_order=row_order)
        ctx.max_ctx_len = self.block_bucket * runner.cache.page_size
        if self.graph is None:
            launches = runner.model.ops.launches
            graph = torch.cuda.CUDAGraph()
            self.capturing = True
            try:
                self.logits = _capture(
                    graph, lambda: runner.model.forward(ctx, runner.cache.views()),
                    runner.graph_pool())
            finally:
                self.capturing = False
            self.graph = graph
            runner.captures += 1
            self.kernels_per_replay = runner.model.ops.launches - launches
        self.graph.replay()
        runner.model.ops.launches += self.kernels_per_replay
        return self.logits
