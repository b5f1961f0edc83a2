"""The flat batch of one step and its index arrays on the device.

A step's tokens, whatever mixture of prompt portions and single decoded tokens they
are, form one batch of N tokens from R requests.  Requests that bring exactly one
token come first, so `n_decode` of them occupy tokens [0, n_decode); the attention
part sends them to the split-KV decode kernel and the rest to the prefill kernel.
All index arrays are packed into one pinned host buffer and reach the device with one
copy.

The reference builds, per forward call, a `StepCtx` with cos/sin rows, a dense
-inf mask [batch, 1, q_len, ctx], a gather plan and flattened cache writes
(src/model.rs:447-533) and requires every item to bring the same number of tokens
(src/model.rs:417-421, 465-469).  Here only positions and tables are sent; the mask
is a comparison inside the attention kernel and the rotation table is resident.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..errors import CacheError


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them
    (0-based) whose logits are wanted."""
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GroupContext:
    block_table: torch.Tensor       # int32 [R, max_blocks]; -1 where a page was released
    slot_mapping: torch.Tensor      # int32 [N]: page * page_size + slot; -1 writes nothing
    max_blocks: int
    page_size: int
    window: Optional[int]


@dataclass
class StepContext:
    ops: object
    n_tokens: int
    n_reqs: int
    n_decode: int                   # requests [0, n_decode) bring one token each
    token_ids: torch.Tensor         # int32 [N]
    positions: torch.Tensor         # int32 [N] absolute position of each token
    token_req: torch.Tensor         # int32 [N] request index of each token
    q_start: torch.Tensor           # int32 [R+1] first token of each request
    ctx_lens: torch.Tensor          # int32 [R] tokens in the cache after this step; 0 = padding
    start_pos: torch.Tensor         # int32 [R] position of the request's first token here
    state_slot: torch.Tensor        # int32 [R]; -1 = padding
    logit_rows: torch.Tensor        # int32 [M] flat token rows whose logits are wanted
    groups: List[GroupContext]
    q_lens: List[int] = field(default_factory=list)        # host copies
    ctx_lens_host: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_len: int = 0
    n_wanted: int = 0               # logit rows that were asked for (the first ones)


def _align(n: int) -> int:
    return (n + 3) & ~3


class BatchBuilder:
    """Packs a step's index arrays; owns the pinned host buffer and the device buffer."""

    def __init__(self, cache, ops, device, pinned: bool):
        self.cache = cache
        self.ops = ops
        self.device = device
        self.pinned = pinned
        self._host = None
        self._dev = None
        self._copied = None         # event: the last copy out of the host buffer is done
        self.last_h2d_bytes = 0

    def _buffers(self, words: int):
        if self._host is None or self._host.numel() < words:
            cap = max(4096, 1 << (words - 1).bit_length())
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=self.pinned)
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._host, self._dev

    def build(self, entries: Sequence[StepEntry], pad_reqs: int = 0,
              pad_blocks: int = 0, buffers=None, row_order: Optional[Sequence[int]] = None,
              pad_mixed: Optional[Sequence[int]] = None) -> StepContext:
        """`entries` must already be ordered single-token requests first.  `pad_reqs` /
        `pad_blocks` pad the request count (with empty requests that every kernel
        skips) and the block-table width, so that a captured launch sequence sees the
        same addresses and sizes; `buffers` = (host, device) to fill instead of the
        builder's own.  `row_order`: the entries' indices in the order in which their wanted
        rows are to come out (the callers' order, when the entries were reordered).

        `pad_mixed` = (D, P, T, W) pads a step of any mixture to fixed sizes: requests
        [0, D) bring one token each (the real single-token entries, then empty ones), requests
        [D, D + P) are the prompt portions (the real ones, then empty ones without tokens; the
        last one owns the tokens that fill the batch up to T and has no context, so every
        kernel computes nothing for them or something nobody reads), and W logit rows come out
        (the wanted ones first)."""
        cache = self.cache
        ps = cache.page_size
        q_lens = [len(e.tokens) for e in entries]
        if any(q == 0 for q in q_lens):
            raise ValueError("a step entry brings no tokens")
        n_decode = 0
        while n_decode < len(entries) and q_lens[n_decode] == 1:
            n_decode += 1
        if any(q == 1 for q in q_lens[n_decode:]):
            raise ValueError("single-token entries must come first")
        r_real = len(entries)
        n_real = sum(q_lens)
        n_want = sum(len(e.want) for e in entries)
        if pad_mixed is not None:
            D, P, T, W = (int(v) for v in pad_mixed)
            n_prefill = r_real - n_decode
            tail = T - D - (n_real - n_decode)           # tokens that only fill the batch
            if pad_reqs or n_decode > D or n_prefill > P or tail < 0 or n_want > W or \
                    (tail > 0 and n_prefill >= P):
                raise ValueError("the step does not fit the padded sizes")
            R, N, M = D + P, T, W
            req_of = list(range(n_decode)) + [D + j for j in range(n_prefill)]
            q_all = [1] * D + q_lens[n_decode:] + [0] * (P - n_prefill)
            if tail:
                q_all[-1] = tail
            dec_pad = D
        else:
            pad = max(0, pad_reqs - r_real)
            if pad and n_decode != r_real:
                raise ValueError("padding is for steps of single tokens only")
            R = r_real + pad
            N = n_real + pad
            # a padded (replayed) step produces the logits of every row, padding included, so
            # that the captured launch sizes do not depend on how many requests are real
            M = N if pad_reqs else n_want
            req_of = list(range(r_real))
            q_all = q_lens + [1] * pad
            dec_pad = n_decode + pad
        rcs = [cache.requests[e.req] for e in entries]
        starts = [rc.computed for rc in rcs]
        ctx = [s + q for s, q in zip(starts, q_lens)]
        for e, rc, c in zip(entries, rcs, ctx):
            if rc.tokens < c:
                raise CacheError(f"request {e.req!r}: {c} tokens but pages for {rc.tokens}")
        n_groups = len(cache.groups)
        max_blocks = []
        for gi in range(n_groups):
            mb = max([-(-c // ps) for c in ctx] + [1])
            max_blocks.append(max(mb, pad_blocks))

        # layout, in int32 words
        off = {}
        cur = 0
        for name, n in (("token_ids", N), ("positions", N), ("token_req", N),
                        ("q_start", R + 1), ("ctx_lens", R), ("start_pos", R),
                        ("state_slot", R), ("logit_rows", M)):
            off[name] = (cur, n)
            cur = _align(cur + n)
        for gi in range(n_groups):
            off[f"slot{gi}"] = (cur, N)
            cur = _align(cur + N)
            off[f"table{gi}"] = (cur, R * max_blocks[gi])
            cur = _align(cur + R * max_blocks[gi])
        host, dev = buffers if buffers is not None else self._buffers(cur)
        if host.numel() < cur:
            raise ValueError("step buffers too small")
        if self._copied is not None:
            self._copied.synchronize()
        h = host.numpy()

        def view(name):
            a, n = off[name]
            return h[a:a + n]

        q_start = np.zeros(R + 1, dtype=np.int64)
        q_start[1:] = np.cumsum(q_all)
        view("q_start")[:] = q_start
        first = [int(q_start[r]) for r in req_of]        # each entry's first token
        tok = view("token_ids")
        pos = view("positions")
        treq = view("token_req")
        tok[:] = 0
        pos[:] = 0
        treq[:] = np.repeat(np.arange(R), q_all)          # empty requests' tokens included
        if n_decode == r_real:                       # single tokens only: no per-request numpy
            tok[:r_real] = [e.tokens[0] for e in entries]
            pos[:r_real] = starts
        else:
            for a, e, s, q in zip(first, entries, starts, q_lens):
                tok[a:a + q] = np.asarray(e.tokens, dtype=np.int64)
                pos[a:a + q] = np.arange(s, s + q)
        cl = view("ctx_lens"); cl[:] = 0
        sp = view("start_pos"); sp[:] = 0
        ss = view("state_slot"); ss[:] = -1
        cl[req_of] = ctx
        sp[req_of] = starts
        ss[req_of] = [rc.slot for rc in rcs]
        rows = view("logit_rows")
        rows[:] = 0
        k = 0
        if pad_reqs:
            rows[:] = np.arange(N)
        emit = range(len(entries)) if row_order is None else row_order
        for i in (emit if not pad_reqs else ()):
            e = entries[i]
            for w in e.want:
                if not 0 <= w < q_lens[i]:
                    raise ValueError(f"request {e.req!r}: wanted place {w} is outside "
                                     f"its {q_lens[i]} tokens")
                rows[k] = first[i] + w
                k += 1
        for gi in range(n_groups):
            mb = max_blocks[gi]
            table = view(f"table{gi}").reshape(R, mb)
            table[:] = -1
            slots = view(f"slot{gi}")
            slots[:] = -1
            for r, a, rc, s, q, c in zip(req_of, first, rcs, starts, q_lens, ctx):
                t = rc.tables[gi].view()
                nb = -(-c // ps)
                table[r, :nb] = t[:nb]
                if q == 1:
                    page = int(t[s // ps])
                    if page < 0:
                        raise CacheError("a token would be written to a released page")
                    slots[a] = page * ps + s % ps
                    continue
                p = np.arange(s, s + q)
                pages = t[p // ps].astype(np.int64)
                if (pages < 0).any():
                    raise CacheError("a token would be written to a released page")
                slots[a:a + q] = pages * ps + p % ps
        dev[:cur].copy_(host[:cur], non_blocking=True)
        self.last_h2d_bytes = cur * 4
        if dev.is_cuda:
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()

        def dview(name):
            a, n = off[name]
            return dev[a:a + n]

        groups = []
        for gi, grp in enumerate(cache.groups):
            groups.append(GroupContext(
                block_table=dview(f"table{gi}").view(R, max_blocks[gi]),
                slot_mapping=dview(f"slot{gi}"), max_blocks=max_blocks[gi],
                page_size=ps, window=grp.need.window))
        ctx_all = [0] * R
        for r, c in zip(req_of, ctx):
            ctx_all[r] = c
        return StepContext(
            ops=self.ops, n_tokens=N, n_reqs=R, n_decode=dec_pad,
            token_ids=dview("token_ids"), positions=dview("positions"),
            token_req=dview("token_req"), q_start=dview("q_start"),
            ctx_lens=dview("ctx_lens"), start_pos=dview("start_pos"),
            state_slot=dview("state_slot"), logit_rows=dview("logit_rows"),
            groups=groups, q_lens=list(q_all), ctx_lens_host=ctx_all,
            max_q_len=max(q_all + [1]), max_ctx_len=max(ctx + [0]), n_wanted=k)
