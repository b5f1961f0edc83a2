"""The engine on the GPU against the plain implementation, in float32 and in bfloat16:
each request alone and whole; most of it in one step and the last 32 tokens one by one;
portions of changing size; mixed batches with few pages; long decoding; first tokens."""
import random

import pytest
import torch

import schedules
from plain_lfm2 import PlainModel
from tiny import write_tiny

pytestmark = pytest.mark.gpu

# float32: the engine and the plain implementation differ by float32 rounding only.
# bfloat16: weights are the same numbers (the files store bfloat16), activations are
# rounded to 8 bits of mantissa (relative 2^-9) at about ten places per layer; over the
# tiny models' 4 to 6 layers this stays below 3 % of the largest logit.
BOUND = {"float32": 1e-5, "bfloat16": 3e-2}


def _requests(vocab, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {n: write_tiny(root, n) for n in ("A", "B")}


@pytest.fixture(scope="module")
def plains(folders):
    return {n: PlainModel(f) for n, f in folders.items()}


_models = {}


def engine(folders, name, dtype):
    from rvllm_b200.engine import load_model
    key = (name, dtype)
    if key not in _models:
        _models[key] = load_model(folders[name], dtype, "cuda")
    return _models[key]


def runner_for(model, page, pages, slots=4, graphs=False):
    from rvllm_b200.engine import ModelRunner, make_cache
    cache = make_cache(model, page, pages, slots)
    return ModelRunner(model, cache, model.ops, use_graphs=graphs)


def compare(got, plain, reqs, dtype):
    worst = 0.0
    for rid, ids in reqs.items():
        ref = plain.logits(ids)
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            err = float((got[(rid, p)] - ref[p]).abs().max()) / scale
            worst = max(worst, err)
            assert err <= BOUND[dtype], (rid, p, err)
            if dtype == "float32":
                assert int(got[(rid, p)].argmax()) == int(ref[p].argmax()), (rid, p)
            else:
                # Greedy tokens in bfloat16, by teacher forcing on the plain tokens: where
                # the plain winner leads the runner-up by more than twice the bound, logits
                # within the bound cannot change the winner, so it has to be the same.
                top = ref[p].topk(2).values
                if float(top[0] - top[1]) > 2 * BOUND[dtype] * scale:
                    assert int(got[(rid, p)].argmax()) == int(ref[p].argmax()), (rid, p)
    return worst


LENGTHS = [5, 17, 31, 70, 9, 100, 64, 33]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("graphs", [False, True])
def test_schedules(folders, plains, name, dtype, schedule, graphs):
    if graphs and schedule in ("whole", "portions"):
        pytest.skip("no single-token steps in this schedule")
    model, cfg = engine(folders, name, dtype)
    reqs = _requests(cfg.vocab_size, LENGTHS, seed=5)
    steps = getattr(schedules, schedule)(reqs)
    page = 8 if name == "A" else 16
    pages = schedules.tokens_held(steps, 64) // page
    runner = runner_for(model, page, pages, graphs=graphs)
    got = schedules.replay(runner, steps)
    assert runner.cache.groups[0].pool.in_use == 0
    compare(got, plains[name], reqs, dtype)
    if schedule == "mixed":
        pool = runner.cache.groups[0].pool
        assert pool.total_allocs > pool.high_water       # pages were used again
    if graphs:
        assert runner.graph_steps > 0


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_schedules_with_full_mantissa_weights(tmp_path_factory, name, schedule):
    """The float32 path on weights that are stored in 32 bits and use all 24 bits of their
    mantissa (the other tests' files hold bfloat16 values, which a product that silently
    rounded its weights to bfloat16 or TF32 would reproduce exactly)."""
    from rvllm_b200.engine import load_model
    key = ("full", name)
    if key not in _models:
        folder = write_tiny(str(tmp_path_factory.mktemp("full32")), name, torch_dtype="float32")
        plain = PlainModel(folder)
        w = plain.w["model.layers.0.conv.in_proj.weight"]
        assert not torch.equal(w, w.bfloat16().float())      # the weights do need 32 bits
        _models[key] = (load_model(folder, "float32", "cuda"), plain)
    (model, cfg), plain = _models[key]
    reqs = _requests(cfg.vocab_size, LENGTHS[:5], seed=6)
    steps = getattr(schedules, schedule)(reqs)
    page = 8 if name == "A" else 16
    runner = runner_for(model, page, schedules.tokens_held(steps, 64) // page,
                        graphs=schedule in ("tail_decode", "mixed"))
    compare(schedules.replay(runner, steps), plain, reqs, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cut_does_not_matter_float32(folders, plains, dtype):
    """The same position computed under different cuts agrees far more closely than the
    bound against the plain implementation."""
    model, cfg = engine(folders, "B", dtype)
    reqs = _requests(cfg.vocab_size, [90, 41], seed=8)
    outs = []
    for schedule in ("whole", "tail_decode", "portions", "mixed"):
        steps = getattr(schedules, schedule)(reqs)
        runner = runner_for(model, 16, schedules.tokens_held(steps, 64) // 16)
        outs.append(schedules.replay(runner, steps))
    bound = 2e-6 if dtype == "float32" else 2e-2
    for key, row in outs[0].items():
        for other in outs[1:]:
            assert float((other[key] - row).abs().max()) <= bound * float(row.abs().max()), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decode(folders, plains, name, dtype):
    """A short prompt, then token by token up to the model's last position."""
    model, cfg = engine(folders, name, dtype)
    n = cfg.max_position_embeddings
    reqs = _requests(cfg.vocab_size, [n], seed=9)
    steps = schedules.tail_decode(reqs, tail=n - 3)
    page = 16
    runner = runner_for(model, page, -(-n // 64) * 64 // page, graphs=True)
    got = schedules.replay(runner, steps)
    compare(got, plains[name], reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens(folders, plains, name, dtype):
    """Prompts of one to five tokens: the first positions, where the convolution state
    is all zeros and a page holds a single key."""
    model, cfg = engine(folders, name, dtype)
    reqs = _requests(cfg.vocab_size, [1, 2, 3, 4, 5], seed=10)
    for fn in (schedules.whole, schedules.tail_decode, schedules.mixed):
        steps = fn(reqs)
        runner = runner_for(model, 16, schedules.tokens_held(steps, 64) // 16)
        compare(schedules.replay(runner, steps), plains[name], reqs, dtype)


def test_position_past_the_table_is_refused(folders):
    model, cfg = engine(folders, "A", "float32")
    from rvllm_b200.engine import StepEntry
    runner = runner_for(model, 16, 32)
    runner.add_request("x")
    with pytest.raises(ValueError, match="exceed"):
        runner.step([StepEntry("x", [1] * (cfg.max_position_embeddings + 1), [0])])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_portion_shapes_are_replayed(folders, plains, dtype):
    """Portions of one fixed size: from its second occurrence a step shape runs as a replayed
    graph; the logits are those of the plain implementation all the same."""
    model, cfg = engine(folders, "B", dtype)
    reqs = _requests(cfg.vocab_size, [64, 64, 64, 48], seed=12)
    steps = schedules.portions(reqs, sizes=(16,))
    runner = runner_for(model, 16, schedules.tokens_held(steps, 64) // 16, graphs=True)
    got = schedules.replay(runner, steps)
    assert runner.graph_steps >= 6 and runner.capture_failures == 0
    compare(got, plains["B"], reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_padded_mixtures_are_replayed(folders, plains, name, dtype):
    """Steps of decoded tokens beside prompt portions of ever different lengths, with only the
    last row of a portion wanted (as the scheduler asks): they are padded to sizes that come
    again, run kernel by kernel the first time and replayed from then on.  The logits are the
    plain implementation's, and bit for bit the same whether a step was replayed or not."""
    from rvllm_b200.engine import StepEntry
    model, cfg = engine(folders, name, dtype)
    rng = random.Random(21)
    page = 8 if name == "A" else 16
    lengths = {"p%d" % i: n for i, n in enumerate((150, 131, 170, 97))}
    reqs = {rid: [rng.randrange(cfg.vocab_size) for _ in range(n + 14)] for rid, n in lengths.items()}

    def schedule():
        """Four requests; prompts fed in portions of changing size while the earlier requests
        decode beside them."""
        steps, done = [], {rid: 0 for rid in reqs}
        live, order = [], list(reqs)
        sizes = [33, 20, 41, 17, 29, 38, 23, 36, 19, 31, 27, 35, 22, 40, 18, 30]
        k = 0
        while order or live:
            if order and (not live or len(steps) % 3 == 0):
                live.append(order.pop(0))
            entries = []
            for rid in list(live):
                left = lengths[rid] - done[rid]
                if left > 0:                                   # a prompt portion
                    n = min(left, sizes[k % len(sizes)]); k += 1
                    entries.append((rid, reqs[rid][done[rid]:done[rid] + n], (n - 1,)))
                    done[rid] += n
                elif done[rid] < len(reqs[rid]):               # a decoded token
                    entries.append((rid, reqs[rid][done[rid]:done[rid] + 1], (0,)))
                    done[rid] += 1
                if done[rid] == len(reqs[rid]):
                    live.remove(rid)
            steps.append(entries)
        return steps

    def run(max_graphs, idle_steps=1024):
        pages = sum(-(-len(v) // page) for v in reqs.values()) + 4
        runner = runner_for(model, page, pages, graphs=True)
        runner.max_mixed_graphs = max_graphs
        runner.mixed_graph_idle_steps = idle_steps
        got, pos = {}, {rid: 0 for rid in reqs}
        for entries in schedule():
            for rid, _, _ in entries:
                if not runner.cache.has(rid):
                    runner.add_request(rid)
            logits = runner.step([StepEntry(*e) for e in entries]).to("cpu", torch.float32)
            for row, (rid, toks, want) in zip(logits, entries):
                got[(rid, pos[rid] + want[0])] = row.clone()
                pos[rid] += len(toks)
        for rid in reqs:
            runner.end_request(rid)
        model.ops.check_status()
        return runner, got

    replayed, got = run(64)
    assert len(replayed._mixed_graphs) > 0 and replayed.graph_steps > 10 and replayed.capture_failures == 0
    few, again = run(2, idle_steps=0)               # room for two: the oldest goes, others come
    assert len(few._mixed_graphs) <= 2 and few.captures > 2 and few.capture_failures == 0
    assert all(torch.equal(got[key], again[key]) for key in got)
    eager, same = run(0)                            # the padded layout, never captured
    assert len(eager._mixed_graphs) == 0
    assert got.keys() == same.keys()
    for key in got:
        assert torch.equal(got[key], same[key]), key
    plain = plains[name]
    for rid, ids in reqs.items():
        ref = plain.logits(ids)
        scale = float(ref.abs().max())
        for (r, p), row in got.items():
            if r == rid:
                assert float((row - ref[p]).abs().max()) / scale <= BOUND[dtype], (rid, p)


def test_scratch_outgrown_after_a_capture(folders, plains):
    """A captured decode step names the split-KV scratch by address.  When a later step
    needs a larger scratch, the old one must stay valid for the older graph: replay it
    afterwards, with other tensors allocated in between, and compare with the plain
    implementation; the tensors allocated in between keep their contents."""
    import gc
    model, cfg = engine(folders, "B", "bfloat16")
    ops = model.ops
    reqs = _requests(cfg.vocab_size, [40], seed=21)
    ids = reqs["r0"]
    from rvllm_b200.engine import StepEntry
    runner = runner_for(model, 16, 8, slots=1, graphs=True)
    runner.add_request("r0")
    runner.step([StepEntry("r0", ids[:30], ())])
    got = {}
    for p in range(30, 34):                         # captures, then replays, bucket (1, 16)
        got[("r0", p)] = runner.step([StepEntry("r0", ids[p:p + 1], (0,))])[0].float().cpu()
    assert runner.graph_steps >= 3
    before = ops._scratch_buffer(1, model.device)
    grown = ops._scratch_buffer(4 * before.numel(), model.device)      # a larger step came
    assert grown.data_ptr() != before.data_ptr()
    del before, grown
    gc.collect()
    torch.cuda.empty_cache()
    canaries = [torch.full((1 << 18,), 7, dtype=torch.int32, device=model.device)
                for _ in range(8)]
    for p in range(34, 40):                         # the old graph again
        got[("r0", p)] = runner.step([StepEntry("r0", ids[p:p + 1], (0,))])[0].float().cpu()
    torch.cuda.synchronize()
    assert all(bool((c == 7).all()) for c in canaries)
    ref = plains["B"].logits(ids)
    scale = float(ref.abs().max())
    for (rid, p), row in got.items():
        assert float((row - ref[p]).abs().max()) / scale <= BOUND["bfloat16"], p
    ops.check_status()
