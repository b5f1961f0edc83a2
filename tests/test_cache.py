"""The cache manager: pages, block tables, groups, window release, state slots.
Invariant under random orders of requests: no page lost, held twice or freed twice."""
import random

import pytest

from rvllm_b200.cache import CacheManager, PagePool
from rvllm_b200.errors import CacheError
from rvllm_b200.parts.base import PagedNeed, StateNeed

FULL = PagedNeed(2, 16, None)
WINDOW = PagedNeed(2, 16, 20)
STATE = StateNeed((2, 8))


def manager(needs, pages=16, page=4, slots=4, cache_of=None):
    return CacheManager(needs, cache_of or [None] * len(needs), page, pages, slots, allocate=False)


def test_pool_hands_out_every_page_once_and_reuses_the_last_freed():
    pool = PagePool(4)
    got = [pool.alloc() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3]
    with pytest.raises(CacheError, match="no free page"):
        pool.alloc()
    pool.free(got[1])
    assert pool.alloc() == got[1]
    assert (pool.total_allocs, pool.high_water, pool.in_use) == (5, 4, 4)


def test_pool_refuses_double_free_and_unknown_pages():
    pool = PagePool(3)
    p = pool.alloc()
    pool.free(p)
    with pytest.raises(CacheError, match="freed twice"):
        pool.free(p)
    with pytest.raises(CacheError, match="does not exist"):
        pool.free(7)


def test_groups_by_need_and_slots_for_state():
    m = manager([STATE, FULL, STATE, WINDOW, FULL, None])
    assert [g.calls for g in m.groups] == [[1, 4], [3]]
    views = m.views()
    assert [v.kind if v else None for v in views] == ["state", "paged", "state", "paged", "paged", None]
    assert (views[1].group, views[3].group, views[4].group) == (0, 1, 0)
    assert sorted(m.states) == [0, 2]
    assert m.bytes_per_token() == 2 * 3 * 2 * 16 * 4


def test_reserve_is_all_or_nothing_and_tables_grow():
    m = manager([FULL], pages=5, page=4)
    a = m.add("a")
    assert m.reserve("a", 9) and len(a.tables[0]) == 3 and a.tokens == 9
    assert m.reserve("a", 12) and len(a.tables[0]) == 3          # same pages cover it
    m.add("b")
    assert not m.reserve("b", 9)                                   # needs 3, only 2 free
    assert m.groups[0].pool.in_use == 3 and m.requests["b"].tables == [[]]
    assert m.reserve("b", 8)
    m.check()
    with pytest.raises(CacheError, match="already live"):
        m.add("a")
    m.free("a")
    assert m.groups[0].pool.in_use == 2
    with pytest.raises(CacheError, match="not live"):
        m.free("a")
    m.check()


def test_freed_pages_are_used_again():
    m = manager([FULL], pages=4, page=4)
    m.add("a"); m.reserve("a", 16)
    first = list(m.requests["a"].tables[0])
    m.free("a")
    m.add("b"); m.reserve("b", 16)
    assert sorted(m.requests["b"].tables[0]) == sorted(first)
    assert m.groups[0].pool.total_allocs == 8 and m.groups[0].pool.high_water == 4


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager([FULL, WINDOW], pages=16, page=4)       # window 20, page 4
    rc = m.add("a")
    m.reserve("a", 40)
    m.advance("a", 40)
    # the next query is at position 40 and sees keys 21..40: pages 0..4 (keys 0..19) go
    assert rc.tables[1][:5] == [-1] * 5 and all(p >= 0 for p in rc.tables[1][5:])
    assert all(p >= 0 for p in rc.tables[0])              # the full group keeps everything
    assert m.groups[1].pool.in_use == 5 and m.groups[0].pool.in_use == 10
    m.check()
    m.reserve("a", 44); m.advance("a", 44)
    assert rc.tables[1][:6] == [-1] * 6
    m.free("a")
    assert m.groups[0].pool.in_use == 0 and m.groups[1].pool.in_use == 0
    m.check()


def test_advance_is_checked():
    m = manager([FULL])
    m.add("a"); m.reserve("a", 8)
    with pytest.raises(CacheError, match="only 8 reserved"):
        m.advance("a", 9)
    m.advance("a", 8)
    with pytest.raises(CacheError, match="cannot move back"):
        m.advance("a", 4)


def test_slots_run_out_and_come_back():
    m = manager([STATE], slots=2)
    a, b = m.add("a"), m.add("b")
    assert {a.slot, b.slot} == {0, 1} and not m.can_add()
    with pytest.raises(CacheError, match="no free state slot"):
        m.add("c")
    m.free("a")
    assert m.add("c").slot == a.slot
    m.check()


def test_a_call_reading_another_calls_cache_shares_its_view():
    m = CacheManager([FULL, None, STATE], [None, 0, None], 4, 8, 2, allocate=True)
    v = m.views()
    assert v[1].kind == "paged" and not v[1].owns and v[0].owns
    assert v[1].k.data_ptr() == v[0].k.data_ptr() and v[1].group == v[0].group
    assert len(m.groups) == 1 and m.groups[0].calls == [0]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    m = manager([FULL, WINDOW, STATE], pages=24, page=4, slots=5)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.can_add():
            m.add(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            more = live[rid] + rng.randint(1, 11)
            if m.reserve(rid, more):
                m.advance(rid, more)
                live[rid] = more
        elif live:
            rid = rng.choice(list(live))
            m.free(rid); del live[rid]
        m.check()
        for g in m.groups:
            assert g.pool.in_use + g.pool.available == g.pool.num_pages
    for rid in list(live):
        m.free(rid)
    assert all(g.pool.in_use == 0 for g in m.groups) and m.slots.in_use == 0
    assert m.groups[0].pool.total_allocs > m.groups[0].pool.num_pages      # reuse happened


def test_padded_mixture_layout():
    """`BatchBuilder.build(pad_mixed=(D, P, T, W))`: the real single-token requests come first
    among D, the real portions first among P, the last (empty) portion owns the filling tokens
    and has no context, nothing that is padding writes a cache slot, and the wanted rows come
    first among W."""
    import numpy as np
    import torch

    from rvllm_b200.cache import CacheManager
    from rvllm_b200.engine import BatchBuilder, StepEntry
    from rvllm_b200.parts.base import PagedNeed, StateNeed
    cache = CacheManager([PagedNeed(2, 16, None), StateNeed((2, 8))], [None, None], 8, 64, 8,
                         dtype=torch.float32, device="cpu", allocate=False)
    builder = BatchBuilder(cache, None, "cpu", pinned=False)
    for rid, done in (("a", 20), ("b", 7), ("c", 0), ("d", 30)):
        cache.add(rid)
        cache.reserve(rid, done)
        cache.advance(rid, done)
    entries = [StepEntry("a", [11], (0,)), StepEntry("b", [12], (0,)),
               StepEntry("c", list(range(100, 119)), ()), StepEntry("d", list(range(200, 205)), (4,))]
    for e in entries:
        cache.reserve(e.req, cache.requests[e.req].computed + len(e.tokens))
    ctx = builder.build(entries, pad_blocks=16, pad_mixed=(4, 4, 64, 8))
    assert (ctx.n_reqs, ctx.n_tokens, ctx.n_decode, ctx.n_wanted) == (8, 64, 4, 3)
    q_start = ctx.q_start.numpy()
    assert q_start.tolist() == [0, 1, 2, 3, 4, 23, 28, 28, 64]
    assert ctx.ctx_lens.numpy().tolist() == [21, 8, 0, 0, 19, 35, 0, 0]
    assert ctx.start_pos.numpy().tolist() == [20, 7, 0, 0, 0, 30, 0, 0]
    slots = ctx.state_slot.numpy()
    assert (slots[[2, 3, 6, 7]] == -1).all() and (slots[[0, 1, 4, 5]] >= 0).all()
    tok = ctx.token_ids.numpy()
    assert tok[:4].tolist() == [11, 12, 0, 0] and tok[4:23].tolist() == list(range(100, 119))
    assert tok[23:28].tolist() == list(range(200, 205)) and (tok[28:] == 0).all()
    assert ctx.positions.numpy()[23:28].tolist() == [30, 31, 32, 33, 34]
    treq = ctx.token_req.numpy()
    assert treq[:4].tolist() == [0, 1, 2, 3] and (treq[4:23] == 4).all() and (treq[28:] == 7).all()
    assert ctx.logit_rows.numpy().tolist() == [0, 1, 27, 0, 0, 0, 0, 0]
    g = ctx.groups[0]
    sm = g.slot_mapping.numpy()
    assert (sm[2:4] == -1).all() and (sm[28:] == -1).all() and (sm[:2] >= 0).all() and (sm[4:28] >= 0).all()
    table = g.block_table.numpy()
    assert table.shape == (8, 16) and (table[[2, 3, 6, 7]] == -1).all()
    assert (table[5, :5] >= 0).all() and (table[5, 5:] == -1).all()
    # sizes that do not fit are refused
    import pytest
    with pytest.raises(ValueError):
        builder.build(entries, pad_mixed=(1, 4, 64, 8))
    with pytest.raises(ValueError):
        builder.build(entries, pad_mixed=(4, 2, 64, 8))        # no empty portion for the filling
    with pytest.raises(ValueError):
        builder.build(entries, pad_mixed=(4, 4, 64, 2))
