"""Each CUDA kernel alone against its plain reference (tests/plain_ops.py), at sizes
other than the engine's: widths that are no power of two, head sizes 48 and 80, groups
of 3, pages of 8, filters of 2 to 5 taps."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

from plain_ops import PlainOps, sample_row, uniform

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from rvllm_b200.kernels import cuda_ops
    return cuda_ops()


def tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def rnd(shape, dtype, gen, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(ops, dtype):
    g = torch.Generator().manual_seed(1)
    table = rnd((777, 200), dtype, g)
    ids = torch.randint(0, 777, (37,), generator=g, dtype=torch.int32)
    ref = torch.empty(37, 200)
    PlainOps().embed(table, ids, ref, 1.5)
    out = torch.empty(37, 200, device="cuda")
    ops.embed(table.cuda(), ids.cuda(), out, 1.5)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [200, 1000, 2048])
def test_add_rmsnorm(ops, dtype, hidden):
    g = torch.Generator().manual_seed(2)
    resid = rnd((19, hidden), torch.float32, g)
    delta = rnd((19, hidden), dtype, g)
    w = 1 + rnd((hidden,), torch.float32, g, 0.05)
    for use_delta in (True, False):
        r_ref, out_ref = resid.clone(), torch.empty(19, hidden, dtype=dtype)
        PlainOps().add_rmsnorm(r_ref, delta if use_delta else None, w, 1e-5, out_ref)
        r_gpu, out = resid.cuda(), torch.empty(19, hidden, dtype=dtype, device="cuda")
        ops.add_rmsnorm(r_gpu, delta.cuda() if use_delta else None, w.cuda(), 1e-5, out)
        assert torch.allclose(r_gpu.cpu(), r_ref, atol=1e-6, rtol=1e-6)
        assert torch.allclose(out.cpu().float(), out_ref.float(), **tol(dtype))
    rows = torch.tensor([3, 18, 0, 3], dtype=torch.int32)
    out_ref = torch.empty(4, hidden, dtype=dtype)
    PlainOps().add_rmsnorm(resid.clone(), delta, w, 1e-6, out_ref, rows)
    r_gpu, out = resid.cuda(), torch.empty(4, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r_gpu, delta.cuda(), w.cuda(), 1e-6, out, rows.cuda())
    assert torch.equal(r_gpu.cpu(), resid)          # stream untouched with a row list
    assert torch.allclose(out.cpu().float(), out_ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ffn", [200, 1024])
def test_swiglu(ops, dtype, ffn):
    g = torch.Generator().manual_seed(3)
    x = rnd((13, 2 * ffn), dtype, g, 2.0)
    ref = torch.empty(13, ffn, dtype=dtype)
    PlainOps().swiglu(x, ref)
    out = torch.empty(13, ffn, dtype=dtype, device="cuda")
    ops.swiglu(x.cuda(), out)
    assert torch.allclose(out.cpu().float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_bias(ops, dtype):
    g = torch.Generator().manual_seed(4)
    x, b = rnd((11, 77), dtype, g), rnd((77,), torch.float32, g)
    ref = x.clone()
    PlainOps().add_bias(ref, b)
    out = x.cuda()
    ops.add_bias(out, b.cuda())
    assert torch.allclose(out.cpu().float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_float32_is_float32(ops, dtype):
    g = torch.Generator().manual_seed(5)
    x, w = rnd((33, 300), dtype, g), rnd((70, 300), dtype, g)
    ref = x.double() @ w.double().t()
    out = ops.linear(x.cuda(), w.cuda(), out_dtype=torch.float32).cpu().double()
    # float32 operands: errors of float32 accumulation only (TF32 would give ~1e-3)
    bound = 2e-5 if dtype == torch.float32 else 2e-5
    assert (out - ref).abs().max() <= bound * ref.abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("norm,rope", [(True, True), (False, True), (True, False)])
def test_qk_norm_rope_write(ops, dtype, norm, rope):
    g = torch.Generator().manual_seed(6)
    nh, nkv, hd, n, ps, pages = 6, 2, 48, 21, 8, 9
    qkv = rnd((n, (nh + 2 * nkv) * hd), dtype, g)
    qw = (1 + rnd((hd,), torch.float32, g, 0.1)) if norm else None
    kw = (1 + rnd((hd,), torch.float32, g, 0.1)) if norm else None
    positions = torch.randint(0, 300, (n,), generator=g, dtype=torch.int32)
    table = None
    if rope:
        ang = torch.arange(300).float().unsqueeze(1) * torch.pow(
            torch.tensor(10000.0), -2.0 * torch.arange(hd // 2).float() / hd)
        table = (ang.cos(), ang.sin())
    slots = torch.randperm(pages * ps, generator=g)[:n].to(torch.int32)
    slots[5] = -1
    kc = rnd((pages, ps, nkv, hd), dtype, g)
    vc = rnd((pages, ps, nkv, hd), dtype, g)
    ref_qkv, ref_k, ref_v = qkv.clone(), kc.clone(), vc.clone()
    PlainOps().qk_norm_rope_write(ref_qkv, nh, nkv, hd, qw, kw, 1e-6, table, positions, slots,
                                  ref_k, ref_v)
    d_qkv, d_k, d_v = qkv.cuda(), kc.cuda(), vc.cuda()
    ops.qk_norm_rope_write(d_qkv, nh, nkv, hd, qw.cuda() if norm else None,
                           kw.cuda() if norm else None, 1e-6,
                           (table[0].cuda(), table[1].cuda()) if rope else None,
                           positions.cuda(), slots.cuda(), d_k, d_v)
    t = tol(dtype)
    assert torch.allclose(d_qkv[:, :nh * hd].cpu().float(), ref_qkv[:, :nh * hd].float(), **t)
    assert torch.allclose(d_k.cpu().float(), ref_k.float(), **t)
    assert torch.equal(d_v.cpu(), ref_v)


@pytest.mark.parametrize("norm,rope", [(True, True), (False, True), (True, False)])
@pytest.mark.parametrize("sizes", [
    # tokens, heads, kv heads, hidden: an odd number of heads in all (the last tile of 128 rows
    # holds one head), K split over a cluster and not, one token and the most the kernel takes
    (8, 6, 2, 512), (1, 3, 1, 72), (16, 5, 2, 4096), (11, 32, 8, 2048),
])
def test_linear_qk_norm_rope_write(ops, sizes, norm, rope):
    """The q|k|v product with norm, rotation and cache write in its epilogue (bfloat16, head
    size 64, few tokens) against the product followed by the plain norm/rotation/write."""
    n, nh, nkv, hidden = sizes
    hd, ps, pages = 64, 8, 9
    g = torch.Generator().manual_seed(14)
    x = rnd((n, hidden), torch.bfloat16, g)
    w = rnd(((nh + 2 * nkv) * hd, hidden), torch.bfloat16, g, 0.05)
    qw = (1 + rnd((hd,), torch.float32, g, 0.1)) if norm else None
    kw = (1 + rnd((hd,), torch.float32, g, 0.1)) if norm else None
    positions = torch.randint(0, 300, (n,), generator=g, dtype=torch.int32)
    table = None
    if rope:
        ang = torch.arange(300).float().unsqueeze(1) * torch.pow(
            torch.tensor(10000.0), -2.0 * torch.arange(hd // 2).float() / hd)
        table = (ang.cos(), ang.sin())
    slots = torch.randperm(pages * ps, generator=g)[:n].to(torch.int32)
    if n > 5:
        slots[5] = -1
    kc = rnd((pages, ps, nkv, hd), torch.bfloat16, g)
    vc = rnd((pages, ps, nkv, hd), torch.bfloat16, g)
    ref_k, ref_v = kc.clone(), vc.clone()
    ref_qkv = PlainOps().linear_qk_norm_rope_write(x, w, nh, nkv, hd, qw, kw, 1e-6, table,
                                                  positions, slots, ref_k, ref_v)
    dev = lambda t: None if t is None else t.cuda()
    results = []
    fused = ops.fuse_qkv_rope
    try:
        for mode in (True, False):
            ops.fuse_qkv_rope = mode
            d_k, d_v = kc.cuda(), vc.cuda()
            d_qkv = ops.linear_qk_norm_rope_write(
                x.cuda(), w.cuda(), nh, nkv, hd, dev(qw), dev(kw), 1e-6,
                (table[0].cuda(), table[1].cuda()) if rope else None, positions.cuda(),
                slots.cuda(), d_k, d_v)
            ops.check_status()
            results.append((d_qkv[:, :nh * hd].cpu().float(), d_k.cpu().float(), d_v.cpu().float()))
    finally:
        ops.fuse_qkv_rope = fused
    scale = float(ref_qkv.float().abs().max())
    for q_out, k_out, v_out in results:
        # the product's rounding to bfloat16 sits before the norm: a last-bit difference of
        # the product is a last-bit difference of the result
        assert (q_out - ref_qkv[:, :nh * hd].float()).abs().max() <= 2e-2 * scale
        assert (k_out - ref_k.float()).abs().max() <= 2e-2 * scale
        assert (v_out - ref_v.float()).abs().max() <= 2e-2 * scale
    # the slot -1 row wrote nothing; untouched slots are untouched
    written = set(int(s_) for s_ in slots.tolist() if s_ >= 0)
    flat_k = results[0][1].reshape(pages * ps, -1)
    for slot in range(pages * ps):
        if slot not in written:
            assert torch.equal(flat_k[slot], kc.float().reshape(pages * ps, -1)[slot])


def attention_case(dtype, g, q_lens, ctx_lens, nh, nkv, hd, ps, window=None, standout=False):
    """A batch with random pages in a shuffled pool.  With `standout`, one far key of
    every request is made to dominate the softmax of its last query."""
    R = len(q_lens)
    n = sum(q_lens)
    blocks = [-(-c // ps) for c in ctx_lens]
    pages = sum(blocks) + 3
    perm = torch.randperm(pages, generator=g).tolist()
    mb = max(blocks)
    table = torch.full((R, mb), -1, dtype=torch.int32)
    k = 0
    for r in range(R):
        for b in range(blocks[r]):
            table[r, b] = perm[k]
            k += 1
    kc = rnd((pages, ps, nkv, hd), dtype, g)
    vc = rnd((pages, ps, nkv, hd), dtype, g)
    q = rnd((n, (nh + 2 * nkv) * hd), dtype, g)
    q_start = [0]
    for ql in q_lens:
        q_start.append(q_start[-1] + ql)
    token_req = [r for r, ql in enumerate(q_lens) for _ in range(ql)]
    if standout:
        for r in range(R):
            p = ctx_lens[r] - 1
            lo = 0 if window is None else max(0, p - window + 1)
            far = lo + (p - lo) // 7           # a key far from the query, inside the window
            t_last = q_start[r + 1] - 1
            page, slot = int(table[r, far // ps]), far % ps
            for h in range(nh):
                qh = q[t_last, h * hd:(h + 1) * hd].float()
                kc[page, slot, h // (nh // nkv)] = (qh / qh.norm() * 6.0).to(dtype)
    n_decode = 0
    while n_decode < R and q_lens[n_decode] == 1:
        n_decode += 1
    ctx = SimpleNamespace(
        n_tokens=n, n_reqs=R, n_decode=n_decode,
        q_start=torch.tensor(q_start, dtype=torch.int32),
        ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32),
        token_req=torch.tensor(token_req, dtype=torch.int32),
        max_ctx_len=max(ctx_lens), max_q_len=max(q_lens))
    group = SimpleNamespace(block_table=table, max_blocks=mb, page_size=ps, window=window)
    return q, kc, vc, ctx, group


def to_cuda(ns):
    return SimpleNamespace(**{k: (v.cuda() if torch.is_tensor(v) else v)
                              for k, v in vars(ns).items()})


ATTN_CASES = [
    # q_lens, ctx_lens, heads, kv heads, head size, page, window
    ([1, 1, 5, 40], [1, 300, 5, 333], 6, 2, 48, 8, None),
    ([1, 7, 2, 64], [700, 7, 130, 64], 3, 1, 80, 16, None),
    ([1, 1, 9, 33], [290, 17, 100, 260], 8, 2, 16, 16, 37),
    ([3], [515], 4, 4, 128, 32, None),
    # head size 64: the decode kernels that stream pages by TMA (pages of 8, 16, 32, 64)
    ([1, 1, 1, 1, 6], [700, 1, 257, 64, 6], 8, 2, 64, 16, None),
    ([1, 1, 1, 2], [300, 255, 9, 130], 12, 4, 64, 8, 100),
    ([1, 1, 1], [1030, 33, 512], 4, 1, 64, 32, None),
    ([1, 1], [400, 70], 2, 2, 64, 64, 129),
    # 32 query heads on one key/value head: two tiles of 16 packed rows per head group
    ([1, 1, 3], [300, 70, 40], 32, 1, 64, 16, None),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTN_CASES)
@pytest.mark.parametrize("standout", [False, True])
def test_paged_attention(ops, dtype, case, standout):
    q_lens, ctx_lens, nh, nkv, hd, ps, window = case
    g = torch.Generator().manual_seed(7)
    q, kc, vc, ctx, group = attention_case(dtype, g, q_lens, ctx_lens, nh, nkv, hd, ps, window,
                                           standout)
    scale = 1.0 / math.sqrt(hd)
    ref = torch.zeros(ctx.n_tokens, nh * hd, dtype=dtype)
    PlainOps().paged_attention(q, nh, nkv, hd, kc, vc, ctx, group, scale, window, ref)
    dq, dk, dv, dctx, dgroup = q.cuda(), kc.cuda(), vc.cuda(), to_cuda(ctx), to_cuda(group)
    t = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    # the dispatching entry (decode kernel for single tokens, prefill kernel for the rest)
    out = torch.full((ctx.n_tokens, nh * hd), float("nan"), dtype=dtype, device="cuda")
    ops.paged_attention(dq, nh, nkv, hd, dk, dv, dctx, dgroup, scale, window, out)
    assert torch.allclose(out.cpu().float(), ref.float(), **t)
    if dtype == torch.bfloat16 and hd == 64:
        # both tensor-core decode kernels by name (the default picks one by the amount of work)
        chosen = ops.decode_kernel
        try:
            for kernel in ("block", "stream"):
                ops.decode_kernel = kernel
                out1 = torch.full((ctx.n_tokens, nh * hd), float("nan"), dtype=dtype, device="cuda")
                ops.paged_attention(dq, nh, nkv, hd, dk, dv, dctx, dgroup, scale, window, out1)
                assert torch.allclose(out1.cpu().float(), ref.float(), **t), kernel
            ops.check_status()
        finally:
            ops.decode_kernel = chosen
    # every token through the general kernel
    out2 = torch.full((ctx.n_tokens, nh * hd), float("nan"), dtype=dtype, device="cuda")
    ops.paged_attention_general(dq, nh, nkv, hd, dk, dv, dctx, dgroup, scale, window, out2)
    assert torch.allclose(out2.cpu().float(), ref.float(), **t)


EDGE_CASES = [
    # q_len, context, window, page: where the window's first key `lo` of the last (and, for a
    # portion, of the first) query falls
    (1, 356, 100, 16),      # lo = 256: a split, tile and page boundary
    (1, 321, 129, 16),      # lo = 192: a tile boundary inside a split
    (1, 258, 50, 16),       # lo = 208: a page boundary inside a tile
    (1, 356, 100, 64),      # lo = 256 with pages of 64
    (8, 356, 100, 16),      # portion: last query lo = 256
    (8, 363, 100, 16),      # portion: first query lo = 256
    (8, 328, 129, 8),       # portion: first query lo = 192, last 199
    (40, 300, 37, 32),      # portion longer than the window
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", EDGE_CASES)
def test_window_edge(ops, dtype, case):
    """The first key of a window must count and the key before it must not.  For the first
    and the last query of each request the key at `lo` is made to dominate the softmax, and
    the key at `lo - 1` is made twice as strong again with a value far from all others: a
    kernel that is off by one at the window's edge returns another vector altogether, not a
    slightly different average.  Every attention kernel that can take the case runs it."""
    q_len, clen, window, ps = case
    nh, nkv, hd = 4, 2, 64
    g = torch.Generator().manual_seed(31)
    q_lens, ctx_lens = [q_len, q_len], [clen, clen - 64]
    q, kc, vc, ctx, group = attention_case(dtype, g, q_lens, ctx_lens, nh, nkv, hd, ps, window)
    q_start = ctx.q_start.tolist()
    for r in range(2):
        for t, p in ((q_start[r], ctx_lens[r] - q_len), (q_start[r + 1] - 1, ctx_lens[r] - 1)):
            lo = p - window + 1
            assert lo >= 1
            for h in range(nh):
                qh = q[t, h * hd:(h + 1) * hd].float()
                for key, strength in ((lo, 6.0), (lo - 1, 12.0)):
                    page, slot = int(group.block_table[r, key // ps]), key % ps
                    kc[page, slot, h // (nh // nkv)] = (qh / qh.norm() * strength).to(dtype)
                    if key == lo - 1:
                        vc[page, slot, h // (nh // nkv)] = 50.0
    scale = 1.0 / math.sqrt(hd)
    ref = torch.zeros(ctx.n_tokens, nh * hd, dtype=dtype)
    PlainOps().paged_attention(q, nh, nkv, hd, kc, vc, ctx, group, scale, window, ref)
    wrong = torch.zeros_like(ref)
    PlainOps().paged_attention(q, nh, nkv, hd, kc, vc, ctx, group, scale, window + 1, wrong)
    assert float((wrong.float() - ref.float()).abs().max()) > 10       # the edge decides the result
    dq, dk, dv, dctx, dgroup = q.cuda(), kc.cuda(), vc.cuda(), to_cuda(ctx), to_cuda(group)
    t = dict(atol=3e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)

    def run(label):
        out = torch.full((ctx.n_tokens, nh * hd), float("nan"), dtype=dtype, device="cuda")
        ops.paged_attention(dq, nh, nkv, hd, dk, dv, dctx, dgroup, scale, window, out)
        assert torch.allclose(out.cpu().float(), ref.float(), **t), label

    run("chosen by size")
    if dtype == torch.bfloat16:
        chosen = ops.decode_kernel, ops.prefill_attention
        try:
            if q_len == 1:
                for kernel in ("block", "stream"):
                    ops.decode_kernel = kernel
                    run(kernel)
            else:
                for kernel in ("tcgen05", "mma"):
                    ops.prefill_attention = kernel
                    run(kernel)
            ops.check_status()
        finally:
            ops.decode_kernel, ops.prefill_attention = chosen
    out2 = torch.full((ctx.n_tokens, nh * hd), float("nan"), dtype=dtype, device="cuda")
    ops.paged_attention_general(dq, nh, nkv, hd, dk, dv, dctx, dgroup, scale, window, out2)
    assert torch.allclose(out2.cpu().float(), ref.float(), **t)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_padding_rows(ops, dtype):
    """Requests with context 0 are padding: zeros out, nothing read."""
    g = torch.Generator().manual_seed(8)
    q, kc, vc, ctx, group = attention_case(dtype, g, [1, 1, 1], [40, 9, 300], 4, 2, 32, 16)
    ctx.ctx_lens[1] = 0
    group.block_table[1] = -1
    out = torch.full((3, 4 * 32), float("nan"), dtype=dtype, device="cuda")
    ops.paged_attention(q.cuda(), 4, 2, 32, kc.cuda(), vc.cuda(), to_cuda(ctx), to_cuda(group),
                        0.17, None, out)
    assert torch.all(out[1] == 0) and torch.isfinite(out).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,bias", [(3, False), (4, True), (2, True), (5, False), (1, False)])
def test_short_conv(ops, dtype, taps, bias):
    g = torch.Generator().manual_seed(9)
    hidden = 200
    q_lens = [1, 1, 2, 5, 40, 70, 3]
    start = [0, 9, 0, 4, 0, 33, 1]
    slots = [5, 2, 7, 0, 3, 6, -1]
    n = sum(q_lens)
    proj = rnd((n, 3 * hidden), dtype, g)
    filt = rnd((hidden, taps), torch.float32, g, 0.5)
    b_in = rnd((3 * hidden,), torch.float32, g, 0.1) if bias else None
    b_conv = rnd((hidden,), torch.float32, g, 0.1) if bias else None
    state = rnd((8, max(taps - 1, 1), hidden), torch.float32, g)[:, :taps - 1].contiguous()
    q_start = [0]
    for ql in q_lens:
        q_start.append(q_start[-1] + ql)
    ctx = SimpleNamespace(n_reqs=len(q_lens), max_q_len=max(q_lens),
                          q_start=torch.tensor(q_start, dtype=torch.int32),
                          state_slot=torch.tensor(slots, dtype=torch.int32),
                          start_pos=torch.tensor(start, dtype=torch.int32))
    ref, ref_state = torch.empty(n, hidden, dtype=dtype), state.clone()
    PlainOps().short_conv(proj, filt, b_in, b_conv, ref_state if taps > 1 else None, ctx, ref)
    out, d_state = torch.empty(n, hidden, dtype=dtype, device="cuda"), state.cuda()
    ops.short_conv(proj.cuda(), filt.cuda(), b_in.cuda() if bias else None,
                   b_conv.cuda() if bias else None, d_state if taps > 1 else None,
                   to_cuda(ctx), out)
    assert torch.allclose(out.cpu().float(), ref.float(), **tol(dtype))
    if taps > 1:
        assert torch.allclose(d_state.cpu(), ref_state, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [3, 4])
def test_short_conv_long_portion_equals_short_portions(ops, dtype, taps):
    """A portion of 150 tokens (the kernel for long portions: eight channels a thread, rows
    requested ahead) gives bit for bit what portions of 40 + 63 + 47 tokens give through the
    state (the kernel for short ones), and the same final state."""
    g = torch.Generator().manual_seed(91)
    hidden, n = 328, 150
    proj = rnd((n, 3 * hidden), dtype, g).cuda()
    filt = rnd((hidden, taps), torch.float32, g, 0.5).cuda()
    b_in = rnd((3 * hidden,), torch.float32, g, 0.1).cuda()
    b_conv = rnd((hidden,), torch.float32, g, 0.1).cuda()

    def run(cuts):
        state = torch.zeros(2, taps - 1, hidden, dtype=torch.float32, device="cuda")
        out = torch.empty(n, hidden, dtype=dtype, device="cuda")
        pos = 0
        for ql in cuts:
            ctx = SimpleNamespace(n_reqs=1, max_q_len=ql,
                                  q_start=torch.tensor([0, ql], dtype=torch.int32, device="cuda"),
                                  state_slot=torch.tensor([1], dtype=torch.int32, device="cuda"),
                                  start_pos=torch.tensor([pos], dtype=torch.int32, device="cuda"))
            ops.short_conv(proj[pos:pos + ql], filt, b_in, b_conv, state, ctx, out[pos:pos + ql])
            pos += ql
        return out, state

    whole, whole_state = run([n])
    parts, parts_state = run([40, 63, 47])
    assert torch.equal(whole, parts)
    assert torch.equal(whole_state, parts_state)
    ref = torch.empty(n, hidden, dtype=dtype)
    ref_state = torch.zeros(2, taps - 1, hidden)
    ctx = SimpleNamespace(n_reqs=1, max_q_len=n, q_start=torch.tensor([0, n], dtype=torch.int32),
                          state_slot=torch.tensor([1], dtype=torch.int32),
                          start_pos=torch.tensor([0], dtype=torch.int32))
    PlainOps().short_conv(proj.cpu(), filt.cpu(), b_in.cpu(), b_conv.cpu(), ref_state, ctx, ref)
    assert torch.allclose(whole.cpu().float(), ref.float(), **tol(dtype))
    assert torch.allclose(whole_state.cpu(), ref_state, atol=1e-6, rtol=1e-6)


def test_argmax_first_maximum_and_nan(ops):
    x = torch.randn(5, 1003)
    x[0, 17] = x[0, 900] = 9.0                 # tie: the first wins
    x[1, :] = float("-inf")                    # nothing above -inf: 0
    x[2, 3] = float("nan")
    x[2, 500] = 8.0
    x[3, 1002] = 50.0                          # the last element of a ragged row
    ref = PlainOps().argmax(x)
    out = ops.argmax(x.cuda()).cpu()
    assert out.tolist() == ref.tolist()
    assert out[0] == 17 and out[1] == 0 and out[2] == 500 and out[3] == 1002


@pytest.mark.parametrize("top_p", [1.0, 0.9, 0.3])
def test_sample_matches_definition(ops, top_p):
    g = torch.Generator().manual_seed(11)
    vocab, rows = 1003, 64
    logits = torch.randn(rows, vocab, generator=g) * 3
    temp = torch.full((rows,), 0.8)
    temp[5] = 0.0                               # a greedy row among sampled ones
    tp = torch.full((rows,), top_p)
    seed = torch.arange(rows, dtype=torch.int64) * 7 + 3
    counter = torch.arange(rows, dtype=torch.int64)
    out = ops.sample(logits.cuda(), temp.cuda(), tp.cuda(), seed.cuda(), counter.cuda()).cpu()
    differ = []
    for m in range(rows):
        want = sample_row(logits[m], float(temp[m]), top_p, int(seed[m]), int(counter[m]))
        if int(out[m]) != want:
            differ.append((m, int(out[m]), want))
    # float32 sums against the definition's float64 sums can move a draw that falls
    # within rounding of a boundary to the neighbouring token; that is rare
    assert len(differ) <= 1, differ
    assert int(out[5]) == int(torch.argmax(logits[5]))


@pytest.mark.parametrize("vocab", [1003, 20000, 65536, 73728, 80000])
def test_sample_on_chip_and_from_memory(ops, vocab):
    """The kernel that keeps a row's probabilities in registers and shared memory and the one
    that re-reads the logits in every pass: rows that fit registers alone, registers and
    shared memory, a row that fills the first kernel to its limit, and (80,000) rows too long
    for it, which then is not used.  They add in different orders, so a draw within float32
    rounding of a boundary may go to the neighbouring kept token: at most one row in twelve may
    differ, and both must follow the definition (float64) with the same allowance."""
    g = torch.Generator().manual_seed(vocab)
    rows = 12
    logits = (torch.randn(rows, vocab, generator=g) * 4)
    temp = 0.5 + torch.rand(rows, generator=g)
    temp[7] = 0.0                                   # a greedy row
    tp = torch.tensor([1.0, 0.95, 0.9, 0.5, 0.3, 0.05] * 2)
    seed = torch.arange(rows, dtype=torch.int64) * 13 + 1
    counter = torch.arange(rows, dtype=torch.int64)
    outs = []
    try:
        for mode in (1, 0):
            ops.lib.rv_sample_set_onchip(mode)
            outs.append(ops.sample(logits.cuda(), temp.cuda(), tp.cuda(), seed.cuda(),
                                   counter.cuda()).cpu())
    finally:
        ops.lib.rv_sample_set_onchip(1)
    assert int((outs[0] != outs[1]).sum()) <= 1
    want = torch.tensor([sample_row(logits[m], float(temp[m]), float(tp[m]), int(seed[m]),
                                    int(counter[m])) for m in range(rows)], dtype=torch.int32)
    for got in outs:
        assert int((got != want).sum()) <= 1, (got.tolist(), want.tolist())
        assert int(got[7]) == int(torch.argmax(logits[7]))


def test_sample_frequencies(ops):
    """Draws over many counters follow softmax(logits / T)."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]])
    n = 4000
    L = logits.repeat(n, 1).cuda()
    out = ops.sample(L, torch.full((n,), 0.7).cuda(), torch.ones(n).cuda(),
                     torch.full((n,), 1234, dtype=torch.int64).cuda(),
                     torch.arange(n, dtype=torch.int64).cuda()).cpu()
    freq = torch.bincount(out.long(), minlength=5).double() / n
    p = torch.softmax(logits[0].double() / 0.7, 0)
    assert (freq - p).abs().max() < 0.03


GEMM_SHAPES = [
    # M, N, K: token counts around the padding steps, widths that are no multiple of the
    # 128-row tile or the 64-element stage, K split over many blocks and not split at all
    (1, 128, 64), (3, 200, 72), (8, 2048, 2048), (16, 6144, 2048), (17, 1000, 520),
    (64, 2048, 8192), (100, 384, 96), (128, 16384, 256), (200, 640, 1096), (256, 130, 2048),
]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(ops, M, N, K, out_dtype):
    g = torch.Generator().manual_seed(12)
    x = rnd((M, K), torch.bfloat16, g)
    w = rnd((N, K), torch.bfloat16, g, 0.05)
    # one entry of x and w made large: a wrong tile, swizzle or K offset cannot hide
    x[M // 2, K // 3] = 40.0
    w[N // 5, K // 3] = 3.0
    ref = x.double() @ w.double().t()
    for _ in range(2):                            # twice: the tickets must be back at zero
        y = ops.linear_tcgen05(x.cuda(), w.cuda(), out_dtype)
        ops.check_status()
        err = (y.double().cpu() - ref).abs().max() / ref.abs().max()
        assert err <= (2e-5 if out_dtype == torch.float32 else 5e-3), float(err)
    # the same numbers whatever rows share the batch: row 0 alone
    y1 = ops.linear_tcgen05(x[:1].contiguous().cuda(), w.cuda(), torch.float32)
    yM = ops.linear_tcgen05(x.cuda(), w.cuda(), torch.float32)
    assert torch.equal(y1[0], yM[0])



@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (3, 200, 72), (8, 2048, 2048), (16, 6144, 2048),
                                   (5, 2048, 8192), (16, 1000, 520), (64, 2048, 8192)])
def test_gemm_tiled_weights(ops, M, N, K):
    """With the weight matrix laid out tile by tile (contiguous bulk copies of two K blocks a
    stage) and with tensor-map boxes of the row-major matrix the MMAs run over the same values in
    the same order: bit-identical results, for tiles and K blocks that the matrix fills only
    partly, K split over a cluster and not; the tiled copy is made once per matrix."""
    g = torch.Generator().manual_seed(13)
    x = rnd((M, K), torch.bfloat16, g).cuda()
    w = rnd((N, K), torch.bfloat16, g, 0.05).cuda()
    was = ops.gemm_tiled
    try:
        ops.gemm_tiled = True
        a = ops.linear_tcgen05(x, w, torch.float32)
        copies = len(ops._tiled)
        a2 = ops.linear_tcgen05(x, w, torch.float32)
        assert len(ops._tiled) == copies                      # the same copy again
        ops.gemm_tiled = False
        b = ops.linear_tcgen05(x, w, torch.float32)
    finally:
        ops.gemm_tiled = was
    ops.check_status()
    assert torch.equal(a, b) and torch.equal(a, a2)
    ref = x.double() @ w.double().t()
    assert float((a.double() - ref).abs().max() / ref.abs().max()) <= 2e-5


PREFILL_CASES = [
    # q_lens, ctx_lens, heads, kv heads, head size, page size, window.  Head size 64: the
    # tcgen05 kernel (128 rows = tokens x heads of a group, tiles of 64 keys): group sizes
    # that do and do not divide 128, one head per group, portions that start in the middle of
    # a context and end inside a tile or a page, several tiles, a window, every page size.
    ([40], [40], 4, 1, 64, 16, None),
    ([128, 3], [128, 3], 8, 2, 64, 16, None),
    ([130], [130], 8, 2, 64, 16, None),
    ([70, 5, 200], [170, 5, 500], 12, 4, 64, 8, None),
    ([33, 64], [400, 64], 6, 2, 64, 32, 100),
    ([50, 2], [50, 700], 3, 3, 64, 64, None),
    ([300], [1000], 5, 1, 64, 16, 257),
    ([257], [257], 1, 1, 64, 16, None),
    ([20, 9], [90, 9], 32, 1, 64, 16, None),      # 4 query tokens per block of 128 rows
    ([15], [75], 7, 1, 64, 8, None),              # 18 tokens x 7 heads = 126 rows, 2 unused
    # few blocks and long contexts: the key tiles of a block are shared out over several blocks
    # and merged (4 parts; 3 parts of which the shorter request fills only some; with a window)
    ([40], [2000], 8, 2, 64, 16, None),
    ([100, 7], [3000, 900], 4, 4, 64, 32, None),
    ([64], [1800], 8, 2, 64, 16, 700),
    ([30], [8100], 8, 2, 64, 16, None),           # 16 parts
]


@pytest.mark.parametrize("case", PREFILL_CASES)
@pytest.mark.parametrize("standout", [False, True])
def test_prefill_attention_kernels(ops, case, standout):
    """Prompt portions through each bfloat16 prefill kernel by name."""
    q_lens, ctx_lens, nh, nkv, hd, ps, window = case
    g = torch.Generator().manual_seed(21)
    q, kc, vc, ctx, group = attention_case(torch.bfloat16, g, q_lens, ctx_lens, nh, nkv, hd, ps,
                                           window, standout)
    scale = 1.0 / math.sqrt(hd)
    ref = torch.zeros(ctx.n_tokens, nh * hd, dtype=torch.bfloat16)
    PlainOps().paged_attention(q, nh, nkv, hd, kc, vc, ctx, group, scale, window, ref)
    dq, dk, dv, dctx, dgroup = q.cuda(), kc.cuda(), vc.cuda(), to_cuda(ctx), to_cuda(group)
    chosen = ops.prefill_attention
    try:
        for kernel in ("tcgen05", "mma", "simt"):
            ops.prefill_attention = kernel
            out = torch.full((ctx.n_tokens, nh * hd), float("nan"), dtype=torch.bfloat16,
                             device="cuda")
            ops.paged_attention(dq, nh, nkv, hd, dk, dv, dctx, dgroup, scale, window, out)
            ops.check_status()
            assert torch.allclose(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2), kernel
    finally:
        ops.prefill_attention = chosen


def test_prefill_attention_tcgen05_is_used(ops):
    """The default choice takes the tcgen05 kernel where it applies (its launch is counted by
    its own library) and refuses nothing it cannot do: other head sizes go to the mma kernel."""
    g = torch.Generator().manual_seed(22)
    for hd, expect in ((64, True), (32, False)):
        q, kc, vc, ctx, group = attention_case(torch.bfloat16, g, [20], [20], 4, 2, hd, 16)
        out = torch.empty(20, 4 * hd, dtype=torch.bfloat16, device="cuda")
        assert ops._tcgen05_prefill_ok(q.cuda(), out, 4, 2, hd, 16) is expect
        ops.paged_attention(q.cuda(), 4, 2, hd, kc.cuda(), vc.cuda(), to_cuda(ctx), to_cuda(group),
                            0.2, None, out)
        assert torch.isfinite(out).all()
