"""The step program (one resident kernel walking a list of operations) against plain torch:
each kind of operation at sizes other than the engine's, and whole decode steps of the tiny
models and of a model with the published head size."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import schedules
from plain_lfm2 import PlainModel
from plain_ops import PlainOps
from tiny import write_tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from rvllm_b200.kernels import cuda_ops
    return cuda_ops()


def rnd(shape, dtype, g, scale=1.0):
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def bf(x):
    return x.to(torch.bfloat16).float()


@pytest.mark.parametrize("sizes", [
    # tokens, hidden, feed-forward, vocabulary: widths that are no multiple of 64 or 128,
    # one token, the most tokens, a product with more tiles than SMs
    (5, 200, 136, 1000), (1, 64, 192, 512), (16, 1024, 2304, 5000), (8, 2048, 8192, 20000),
])
def test_stream_products_swiglu_logits(ops, sizes):
    """embedding -> norm -> gate|up product -> SwiGLU -> down product -> norm -> head -> logits,
    twice in a row on the same program (the meeting counters must be back at zero)."""
    from rvllm_b200.kernels.program import Embedding, StepProgram
    m, h, f, v = sizes
    g = torch.Generator().manual_seed(m * 1000 + h)
    table = rnd((v, h), torch.bfloat16, g)
    w1 = (1 + rnd((h,), torch.float32, g, 0.1))
    w2 = (1 + rnd((h,), torch.float32, g, 0.1))
    gate_up = rnd((2 * f, h), torch.bfloat16, g, h ** -0.5)
    down = rnd((h, f), torch.bfloat16, g, f ** -0.5)
    head = rnd((v, h), torch.bfloat16, g, h ** -0.5)
    ids = torch.randint(0, v, (16,), generator=g, dtype=torch.int32)
    eps = 1e-5
    dev = lambda t: t.cuda()
    d = {k: dev(t) for k, t in dict(table=table, w1=w1, w2=w2, gate_up=gate_up, down=down,
                                    head=head, ids=ids).items()}
    prog = StepProgram(ops, "cuda", m, h)
    for dry in (True, False):
        prog.begin(dry)
        rows = prog.add_norm(Embedding(d["table"], 1.0, d["ids"]), d["w1"], eps)
        act = prog.swiglu(prog.gemm(rows, d["gate_up"]), f)
        rows2 = prog.add_norm(prog.gemm(act, d["down"]), d["w2"], eps)
        prog.logits(prog.gemm(rows2, d["head"]))
    prog.finish()
    # plain: the same roundings (rows to bfloat16 before a product, float32 everywhere else)
    x = table[ids[:m].long()].float()
    r1 = 1.0 / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    gu = (bf(x * w1) @ gate_up.float().t()) * r1
    act_ref = bf(gu[:, :f] / (1 + torch.exp(-gu[:, :f])) * gu[:, f:])
    x2 = x + act_ref @ down.float().t()
    r2 = 1.0 / torch.sqrt(x2.pow(2).mean(-1, keepdim=True) + eps)
    want = (bf(x2 * w2) @ head.float().t()) * r2
    for _ in range(2):
        got = prog.run()[:m].float().cpu()
        ops.check_status()
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 4e-3 * scale
    assert torch.allclose(prog.resid[:m].cpu(), x2, atol=1e-3 * float(x2.abs().max()), rtol=0)


@pytest.mark.parametrize("taps,bias", [(3, False), (4, True), (2, False), (1, False)])
def test_conv_operation(ops, taps, bias):
    """in_proj product -> gated convolution with state -> out_proj product, into the stream:
    first tokens (state zero), later tokens (state read and shifted), a padding request."""
    from rvllm_b200.kernels.program import Embedding, StepProgram
    m, h, v = 6, 136, 300
    g = torch.Generator().manual_seed(taps)
    table = rnd((v, h), torch.bfloat16, g)
    w_norm = 1 + rnd((h,), torch.float32, g, 0.1)
    w_next = 1 + rnd((h,), torch.float32, g, 0.1)
    w_in = rnd((3 * h, h), torch.bfloat16, g, h ** -0.5)
    w_out = rnd((h, h), torch.bfloat16, g, h ** -0.5)
    filt = rnd((h, taps), torch.float32, g, 0.5)
    b_in = rnd((3 * h,), torch.float32, g, 0.1) if bias else None
    b_conv = rnd((h,), torch.float32, g, 0.1) if bias else None
    b_out = rnd((h,), torch.float32, g, 0.1) if bias else None
    state = rnd((8, max(taps - 1, 1), h), torch.float32, g)[:, :taps - 1].contiguous()
    ids = torch.randint(0, v, (16,), generator=g, dtype=torch.int32)
    slots = torch.tensor([5, 2, -1, 0, 3, 7] + [-1] * 10, dtype=torch.int32)
    start = torch.tensor([0, 9, 0, 4, 0, 1] + [0] * 10, dtype=torch.int32)
    eps = 1e-6
    cu = lambda t: None if t is None else t.cuda()
    d_state = state.cuda()
    ctx = SimpleNamespace(state_slot=slots.cuda(), start_pos=start.cuda())
    prog = StepProgram(ops, "cuda", m, h)
    keep = [cu(t) for t in (table, w_norm, w_in, filt, b_in, b_conv, w_out, b_out, w_next, ids)]
    for dry in (True, False):
        prog.begin(dry)
        rows = prog.add_norm(Embedding(keep[0], 1.0, keep[9]), keep[1], eps)
        y = prog.conv(prog.gemm(rows, keep[2]), keep[3], keep[4], keep[5],
                      d_state if taps > 1 else None, ctx)
        out = prog.gemm(y, keep[6])
        out.bias = keep[7]
        prog.add_norm(out, keep[8], eps)
    prog.finish()
    prog.run()
    ops.check_status()
    # plain
    x = table[ids[:m].long()].float()
    r = 1.0 / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    proj = (bf(x * w_norm) @ w_in.float().t()) * r
    ref_state = state.clone()
    pctx = SimpleNamespace(n_reqs=m, max_q_len=1, q_start=torch.arange(m + 1, dtype=torch.int32),
                           state_slot=slots[:m], start_pos=start[:m])
    y_ref = torch.empty(m, h)
    PlainOps().short_conv(proj, filt, b_in, b_conv, ref_state if taps > 1 else None, pctx, y_ref)
    mixed = bf(y_ref) @ w_out.float().t()
    if bias:
        mixed = mixed + b_out
    want = x + mixed
    got = prog.resid[:m].cpu()
    assert float((got - want).abs().max()) <= 4e-3 * float(want.abs().max())
    if taps > 1:
        assert torch.allclose(d_state.cpu(), ref_state, atol=2e-3 * float(ref_state.abs().max()), rtol=0)


@pytest.mark.parametrize("sizes", [
    # heads, kv heads, head size, hidden, norm, rotation
    (6, 2, 16, 96, True, True), (3, 1, 32, 96, True, True), (32, 8, 64, 512, True, True),
    (4, 4, 128, 256, False, True), (5, 1, 48, 80, True, False),
])
def test_qk_operation(ops, sizes):
    """q|k|v product -> per-head norm, rotation, query rows out, keys and values into their
    slots; a token with slot -1 writes nothing."""
    from rvllm_b200.kernels.program import Embedding, StepProgram
    nh, nkv, hd, h, norm, rope = sizes
    m, v, ps, pages = 7, 200, 8, 9
    g = torch.Generator().manual_seed(hd + nh)
    table = rnd((v, h), torch.bfloat16, g)
    w_norm = 1 + rnd((h,), torch.float32, g, 0.1)
    w_qkv = rnd(((nh + 2 * nkv) * hd, h), torch.bfloat16, g, h ** -0.5)
    qw = (1 + rnd((hd,), torch.float32, g, 0.1)) if norm else None
    kw = (1 + rnd((hd,), torch.float32, g, 0.1)) if norm else None
    ids = torch.randint(0, v, (16,), generator=g, dtype=torch.int32)
    positions = torch.randint(0, 300, (16,), generator=g, dtype=torch.int32)
    tab = None
    if rope:
        ang = torch.arange(300).float().unsqueeze(1) * torch.pow(
            torch.tensor(10000.0), -2.0 * torch.arange(hd // 2).float() / hd)
        tab = (ang.cos().contiguous(), ang.sin().contiguous())
    slots = torch.full((16,), -1, dtype=torch.int32)
    slots[:m] = torch.randperm(pages * ps, generator=g)[:m].to(torch.int32)
    slots[3] = -1
    kc = rnd((pages, ps, nkv, hd), torch.bfloat16, g)
    vc = rnd((pages, ps, nkv, hd), torch.bfloat16, g)
    eps = 1e-5
    cu = lambda t: None if t is None else t.cuda()
    d_k, d_v = kc.cuda(), vc.cuda()
    keep = [cu(t) for t in (table, w_norm, w_qkv, qw, kw, ids, positions, slots)]
    dtab = (tab[0].cuda(), tab[1].cuda()) if rope else None
    prog = StepProgram(ops, "cuda", m, h)
    q_buf = None
    for dry in (True, False):
        prog.begin(dry)
        rows = prog.add_norm(Embedding(keep[0], 1.0, keep[5]), keep[1], eps)
        q_buf = prog.qk(prog.gemm(rows, keep[2]), nh, nkv, hd, keep[3], keep[4], 1e-6, dtab,
                        keep[6], keep[7], d_k, d_v)
    prog.finish()
    prog.run()
    ops.check_status()
    x = table[ids[:m].long()].float()
    r = 1.0 / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    qkv = (bf(x * w_norm) @ w_qkv.float().t()) * r
    ref_k, ref_v = kc.float(), vc.float()
    PlainOps().qk_norm_rope_write(qkv, nh, nkv, hd, qw, kw, 1e-6, tab, positions[:m], slots[:m],
                                  ref_k, ref_v)
    scale = float(qkv.abs().max())
    assert float((q_buf[:m, :nh * hd].float().cpu() - qkv[:, :nh * hd]).abs().max()) <= 1e-2 * scale
    assert float((d_k.float().cpu() - ref_k).abs().max()) <= 1e-2 * max(scale, float(ref_k.abs().max()))
    assert float((d_v.float().cpu() - ref_v).abs().max()) <= 1e-2 * max(scale, float(ref_v.abs().max()))
    # the token with slot -1 wrote nothing, and no other slot was touched
    written = {int(s) for s in slots[:m].tolist() if s >= 0}
    flat, orig = d_k.float().cpu().reshape(pages * ps, -1), kc.float().reshape(pages * ps, -1)
    for slot in range(pages * ps):
        if slot not in written:
            assert torch.equal(flat[slot], orig[slot])


@pytest.mark.parametrize("name", ["A", "B"])
def test_decode_steps_run_as_a_program(tmp_path_factory, name, monkeypatch):
    """Replayed single-token steps of the tiny models in bfloat16 are carried out by a step
    program (not by a silent fallback to one launch per operation) and agree with the plain
    implementation."""
    from rvllm_b200.engine import ModelRunner, load_model, make_cache
    monkeypatch.setenv("RVLLM_STEP_PROGRAM", "1")
    folder = write_tiny(str(tmp_path_factory.mktemp("prog")), name)
    plain = PlainModel(folder)
    model, cfg = load_model(folder, "bfloat16", "cuda")
    rng = random.Random(3)
    reqs = {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n)]
            for i, n in enumerate((40, 9, 70, 33, 17))}
    steps = schedules.mixed(reqs, decode_tail=20)
    page = 8 if name == "A" else 16
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, 4)
    runner = ModelRunner(model, cache, model.ops, use_graphs=True)
    got = schedules.replay(runner, steps)
    model.ops.check_status()
    programs = [g.program for g in runner._graphs.values()]
    assert programs and all(p is not None for p in programs)
    for rid, ids in reqs.items():
        ref = plain.logits(ids)
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            assert float((got[(rid, p)] - ref[p]).abs().max()) <= 3e-2 * scale, (rid, p)


def test_program_and_kernel_path_agree_at_published_head_size(tmp_path_factory):
    """LFM2-350M widths, four layers: the same decode steps through the step program and,
    with RVLLM_STEP_PROGRAM=0, through one launch per operation."""
    import os
    from rvllm_b200.config import config_from_dict
    from rvllm_b200.engine import ModelRunner, StepEntry, load_model, make_cache
    from rvllm_b200.weights import write_random_model
    from test_gpu_sizes import BF16_BOUND_4_LAYERS, LONG
    cfg = config_from_dict(LONG)
    folder = write_random_model(str(tmp_path_factory.mktemp("prog350")), cfg, 4)
    plain = PlainModel(folder)
    model, cfg = load_model(folder, "bfloat16", "cuda")
    rng = random.Random(5)
    prompts = {k: [rng.randrange(4096) for _ in range(n)] for k, n in (("a", 300), ("b", 41), ("c", 150))}
    outs = {}
    for mode in ("1", "0"):
        os.environ["RVLLM_STEP_PROGRAM"] = mode
        try:
            cache = make_cache(model, 16, 64, 4)
            runner = ModelRunner(model, cache, model.ops, use_graphs=True)
            rows = {}
            for k, ids in prompts.items():
                runner.add_request(k)
                runner.step([StepEntry(k, ids[:-12], ())])
            for j in range(12):
                entries = [StepEntry(k, [ids[len(ids) - 12 + j]], (0,)) for k, ids in prompts.items()]
                logits = runner.step(entries).float().cpu()
                for row, e in zip(logits, entries):
                    rows[(e.req, len(prompts[e.req]) - 12 + j)] = row
            model.ops.check_status()
            used = [g.program is not None for g in runner._graphs.values()]
            assert used and all(used) == (mode == "1")
            outs[mode] = rows
        finally:
            os.environ.pop("RVLLM_STEP_PROGRAM", None)
    for (rid, p), row in outs["1"].items():
        ref = plain.logits(prompts[rid][:p + 1])[-1]
        scale = float(ref.abs().max())
        assert float((row - ref).abs().max()) <= BF16_BOUND_4_LAYERS * scale, (rid, p)
        assert float((row - outs["0"][(rid, p)]).abs().max()) <= BF16_BOUND_4_LAYERS * scale
