"""The published LFM2-350M sizes (16 layers, attention at [2,5,8,10,12,14], hidden 1024, 16
query heads, 8 KV heads, head size 64, feed-forward 6656 adjusted to 4608, filter length 3,
vocabulary 65536, tied head) with random weights: float32 logits against the plain
implementation within 1e-5, identical greedy tokens, under whole, chunked and mixed schedules;
bfloat16 within its bound.  The tiny models cannot show faults that need a real head size,
a vocabulary of 65,536 or rows of 1,024 values."""
import random

import pytest
import torch

import schedules
from plain_lfm2 import PlainModel
from rvllm_b200.config import config_from_dict
from rvllm_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

LFM2_350M = {
    "architectures": ["Lfm2ForCausalLM"],
    "num_hidden_layers": 16, "full_attn_idxs": [2, 5, 8, 10, 12, 14],
    "hidden_size": 1024, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 64,
    "block_ff_dim": 6656, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "conv_L_cache": 3, "conv_bias": False, "vocab_size": 65536, "rope_theta": 1000000.0,
    "max_position_embeddings": 4096, "norm_eps": 1e-5, "tie_embedding": True,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 7,
}


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    cfg = config_from_dict(LFM2_350M)
    assert cfg.ffn_dim == 4608
    folder = write_random_model(str(tmp_path_factory.mktemp("lfm2_350m")), cfg, 0)
    plain = PlainModel(folder)
    rng = random.Random(0)
    reqs = {f"s{i}": [rng.randrange(65536) for _ in range(n)] for i, n in enumerate((150, 37, 90))}
    refs = {k: plain.logits(v) for k, v in reqs.items()}
    return folder, reqs, refs


# bfloat16 bound for this depth.  Activations are rounded to 8 bits of mantissa (relative
# error up to 2^-9) at about ten places per layer; independent roundings add like a random
# walk, so after L layers the error of a logit relative to the largest one is about
# sqrt(10 L) * 2^-9, and the bound allows twice that: 3.0 % for the tiny models' 6 layers (the
# bound used there), 4.9 % for the 16 layers here.
BF16_BOUND_16_LAYERS = 2 * (10 * 16) ** 0.5 * 2 ** -9


@pytest.mark.parametrize("dtype,bound", [("float32", 1e-5), ("bfloat16", BF16_BOUND_16_LAYERS)])
def test_real_sizes_against_plain(setup, dtype, bound):
    from rvllm_b200.engine import ModelRunner, load_model, make_cache
    folder, reqs, refs = setup
    model, cfg = load_model(folder, dtype, "cuda")
    worst = 0.0
    for name in ("whole", "portions", "mixed"):
        steps = schedules.tail_decode(reqs, 8) if name == "tail" else getattr(schedules, name)(reqs)
        cache = make_cache(model, 16, schedules.tokens_held(steps, 64) // 16, 4)
        runner = ModelRunner(model, cache, model.ops, use_graphs=True)
        got = schedules.replay(runner, steps)
        for rid, ids in reqs.items():
            ref = refs[rid]
            scale = float(ref.abs().max())
            for p in range(len(ids)):
                err = float((got[(rid, p)] - ref[p]).abs().max()) / scale
                worst = max(worst, err)
                assert err <= bound, (name, rid, p, err)
                if dtype == "float32":
                    assert int(got[(rid, p)].argmax()) == int(ref[p].argmax()), (name, rid, p)
    model.ops.check_status()
    print(f"{dtype}: worst relative error {worst:.2e}")


@pytest.mark.parametrize("decode_kernel,prefill_kernel", [("stream", "tcgen05"), ("block", "mma")])
def test_real_sizes_each_attention_kernel(setup, decode_kernel, prefill_kernel):
    """The same in bfloat16 with the attention kernels named instead of chosen by size: the
    short test contexts would otherwise never reach the stream decode kernel."""
    from rvllm_b200.engine import ModelRunner, load_model, make_cache
    folder, reqs, refs = setup
    model, cfg = load_model(folder, "bfloat16", "cuda")
    ops = model.ops
    chosen = ops.decode_kernel, ops.prefill_attention
    ops.decode_kernel, ops.prefill_attention = decode_kernel, prefill_kernel
    try:
        steps = schedules.mixed(reqs)
        cache = make_cache(model, 16, schedules.tokens_held(steps, 64) // 16, 4)
        runner = ModelRunner(model, cache, ops, use_graphs=True)
        got = schedules.replay(runner, steps)
        ops.check_status()
    finally:
        ops.decode_kernel, ops.prefill_attention = chosen
    for rid, ids in reqs.items():
        ref = refs[rid]
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            err = float((got[(rid, p)] - ref[p]).abs().max()) / scale
            assert err <= BF16_BOUND_16_LAYERS, (rid, p, err)


def test_decode_step_fuses_qk_rope_into_the_product(setup):
    """A decode step at these sizes (head size 64, bfloat16) runs the q/k norm + rotation +
    cache write inside the q|k|v product: one launch less per attention layer than with the
    separate kernel, and the same logits within bfloat16 rounding."""
    from rvllm_b200.engine import ModelRunner, StepEntry, load_model, make_cache
    folder, reqs, refs = setup
    model, cfg = load_model(folder, "bfloat16", "cuda")
    ops = model.ops
    ids = reqs["s1"]
    fused = ops.fuse_qkv_rope
    out, launches = {}, {}
    try:
        for mode in (True, False):
            ops.fuse_qkv_rope = mode
            cache = make_cache(model, 16, 8, 1)
            runner = ModelRunner(model, cache, ops, use_graphs=False)
            runner.add_request("r")
            runner.step([StepEntry("r", ids[:-2], ())])
            # the first single-token step also lays the matrices out tile by tile (one launch
            # each, once): the launches are counted on the second
            runner.step([StepEntry("r", ids[-2:-1], (0,))])
            before = ops.launches
            out[mode] = runner.step([StepEntry("r", ids[-1:], (0,))])[0].float().cpu()
            launches[mode] = ops.launches - before
    finally:
        ops.fuse_qkv_rope = fused
    ops.check_status()
    assert launches[False] - launches[True] == len(LFM2_350M["full_attn_idxs"])
    scale = float(out[False].abs().max())
    assert float((out[True] - out[False]).abs().max()) <= BF16_BOUND_16_LAYERS * scale


# ---- the widths the benchmark runs at ---------------------------------------------------------

def _widths(hidden, heads, ff):
    """The published layer widths of LFM2-1.2B / 700M with the depth cut to four layers (two
    convolution, two attention): every matrix shape, head count and the vocabulary are the
    full model's; only the number of layers is smaller, to keep the plain side quick."""
    return {
        "architectures": ["Lfm2ForCausalLM"],
        "num_hidden_layers": 4, "full_attn_idxs": [1, 3],
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": 8,
        "head_dim": 64, "block_ff_dim": ff, "block_auto_adjust_ff_dim": True,
        "block_multiple_of": 256, "conv_L_cache": 3, "conv_bias": False, "vocab_size": 65536,
        "rope_theta": 1000000.0, "max_position_embeddings": 4096, "norm_eps": 1e-5,
        "tie_embedding": True, "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 7,
    }


WIDTHS = {"1.2B": (_widths(2048, 32, 12288), 8192), "700M": (_widths(1536, 24, 10240), 6912)}
BF16_BOUND_4_LAYERS = 2 * (10 * 4) ** 0.5 * 2 ** -9


@pytest.fixture(scope="module", params=sorted(WIDTHS))
def wide(request, tmp_path_factory):
    data, ffn = WIDTHS[request.param]
    cfg = config_from_dict(data)
    assert cfg.ffn_dim == ffn
    folder = write_random_model(str(tmp_path_factory.mktemp("lfm2_wide")), cfg, 2)
    plain = PlainModel(folder)
    rng = random.Random(3)
    reqs = {f"w{i}": [rng.randrange(65536) for _ in range(n)]
            for i, n in enumerate((131, 40, 77, 18))}
    refs = {k: plain.logits(v) for k, v in reqs.items()}
    return request.param, folder, reqs, refs


@pytest.mark.parametrize("dtype,bound", [("float32", 1e-5), ("bfloat16", BF16_BOUND_4_LAYERS)])
def test_published_widths_against_plain(wide, dtype, bound):
    """Hidden 2048 with 32/8 heads and hidden 1536 with 24/8 heads (three query heads per
    key/value head; 12 and 54 weight tiles per product): whole, in portions and mixed with
    up to four live requests, in float32 (1e-5, same greedy token at every position) and in
    bfloat16; then a few replayed decode steps of all four requests together."""
    from rvllm_b200.engine import ModelRunner, load_model, make_cache
    size, folder, reqs, refs = wide
    model, cfg = load_model(folder, dtype, "cuda")
    worst = 0.0
    for name in ("whole", "portions", "mixed"):
        steps = getattr(schedules, name)(reqs)
        cache = make_cache(model, 16, schedules.tokens_held(steps, 64) // 16, 4)
        runner = ModelRunner(model, cache, model.ops, use_graphs=True)
        got = schedules.replay(runner, steps)
        for rid, ids in reqs.items():
            ref = refs[rid]
            scale = float(ref.abs().max())
            for p in range(len(ids)):
                err = float((got[(rid, p)] - ref[p]).abs().max()) / scale
                worst = max(worst, err)
                assert err <= bound, (size, name, rid, p, err)
                top = ref[p].topk(2).values
                if dtype == "float32" or float(top[0] - top[1]) > 2 * bound * scale:
                    assert int(got[(rid, p)].argmax()) == int(ref[p].argmax()), (name, rid, p)
    model.ops.check_status()
    print(f"{size} {dtype}: worst relative error {worst:.2e}")


# ---- long contexts: the regime the benchmark's numbers are measured in -------------------------

LONG = {
    "architectures": ["Lfm2ForCausalLM"],
    "num_hidden_layers": 4, "full_attn_idxs": [1, 3],
    "hidden_size": 1024, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 64,
    "block_ff_dim": 6656, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "conv_L_cache": 3, "conv_bias": False, "vocab_size": 4096, "rope_theta": 1000000.0,
    "max_position_embeddings": 4096, "norm_eps": 1e-5, "tie_embedding": True,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 7,
}


@pytest.fixture(scope="module")
def long_setup(tmp_path_factory):
    """LFM2-350M widths, four layers, a small vocabulary.  The q norm weights are scaled by
    three, so attention scores spread over some ten units and each query's softmax rests
    on a few dozen keys anywhere in its context (the largest weight is around a tenth): a key left out at a page, tile or split
    boundary, or a wrong page among the two hundred of a long request, moves the logits
    far beyond rounding (with unscaled random weights every key weighs 1/3000)."""
    import os
    from plain_lfm2 import read_safetensors
    from rvllm_b200.weights import write_safetensors
    cfg = config_from_dict(LONG)
    folder = write_random_model(str(tmp_path_factory.mktemp("lfm2_long")), cfg, 5)
    path = os.path.join(folder, "model.safetensors")
    tensors = read_safetensors(path, torch.bfloat16)
    for name in tensors:
        if name.endswith("q_layernorm.weight"):
            tensors[name] = (tensors[name].float() * 3.0).to(torch.bfloat16)
    write_safetensors(path, tensors)
    plain = PlainModel(folder)
    rng = random.Random(8)
    lengths = {"long": 3130, "a": 1590, "b": 300, "c": 90}
    reqs = {k: [rng.randrange(4096) for _ in range(n)] for k, n in lengths.items()}
    refs = {k: plain.logits(v) for k, v in reqs.items()}
    # What a lost page would do: the plain logits of the long request with the sixteen keys
    # [1024, 1040) hidden from every later query.
    import plain_lfm2
    honest = plain_lfm2.causal_mask

    def one_page_hidden(n, window, dtype):
        mask = honest(n, window, dtype)
        mask[1040:, 1024:1040] = float("-inf")
        return mask
    plain_lfm2.causal_mask = one_page_hidden
    try:
        damaged = plain.logits(reqs["long"])
    finally:
        plain_lfm2.causal_mask = honest
    return folder, reqs, refs, damaged


# Scores of the sharpened model reach +-10, so the 8-bit rounding of q and k moves a softmax
# weight by several per cent where it moves it by a few tenths of a per cent with plain random
# weights: the bfloat16 bound is twice that of a four-layer model.  It still sits far below
# what one lost page does (checked in the test: more than twice the bound).
LONG_BOUNDS = [("float32", 1e-5), ("bfloat16", 2 * BF16_BOUND_4_LAYERS)]


@pytest.mark.parametrize("dtype,bound", LONG_BOUNDS)
def test_long_context_across_the_2048_boundary(long_setup, dtype, bound):
    """Four live requests, two of them past 1,500 tokens: prompts in portions of 512 beside
    each other, then 70 replayed single-token steps in which the longest request goes from
    2,040 to 2,110 tokens: the block table's padded width goes from 128 to 256 pages (a new
    graph), the decode splits from 8 to 16, and with four requests the work passes the size
    at which the decode kernel is chosen differently.  Then the three shorter requests end,
    the long one takes another 1,000 tokens in portions of 512 (on the pages the others gave
    back) and decodes to 3,130.  The kernels are chosen by size, as in serving."""
    from rvllm_b200.engine import ModelRunner, StepEntry, load_model, make_cache
    folder, reqs, refs, damaged = long_setup
    model, cfg = load_model(folder, dtype, "cuda")
    ops = model.ops
    assert ops.decode_kernel == "auto" and ops.prefill_attention == "auto"
    tail = 70
    first = {"long": 2110, "a": 1590, "b": 300, "c": 90}       # tokens of the first stage
    total = sum(-(-n // 64) * 64 for n in first.values())
    cache = make_cache(model, 16, total // 16, 4)
    pool = cache.groups[0].pool
    runner = ModelRunner(model, cache, ops, use_graphs=True)
    got = {}
    done = {k: 0 for k in reqs}
    for k in reqs:
        runner.add_request(k)

    def prompts(upto):
        """Portions of 512 of every request that is more than `tail` tokens short of `upto`."""
        while True:
            entries = []
            for k, ids in reqs.items():
                left = upto.get(k, 0) - tail - done[k]
                if left > 0:
                    n = min(512, left)
                    entries.append(StepEntry(k, ids[done[k]:done[k] + n], (n - 1,)))
            if not entries:
                return
            logits = runner.step(entries).float().cpu()
            for row, e in zip(logits, entries):
                done[e.req] += len(e.tokens)
                got[(e.req, done[e.req] - 1)] = row
            cache.check()

    def decode(names, steps):
        for _ in range(steps):
            entries = [StepEntry(k, reqs[k][done[k]:done[k] + 1], (0,)) for k in names]
            logits = runner.step(entries).float().cpu()
            for row, e in zip(logits, entries):
                got[(e.req, done[e.req])] = row
                done[e.req] += 1
            buckets.add(max(key[1] for key in runner._graphs))

    buckets = set()
    prompts(first)
    decode(list(reqs), tail)
    assert buckets == {128, 256}                       # the table's width changed on the way
    assert runner.graph_steps >= tail - 2
    assert done == first
    for k in ("a", "b", "c"):
        runner.end_request(k)
    allocs = pool.total_allocs
    prompts({"long": len(reqs["long"])})
    decode(["long"], len(reqs["long"]) - done["long"])
    assert done["long"] == 3130 and pool.total_allocs > allocs and pool.high_water <= total // 16
    runner.end_request("long")
    cache.check()
    ops.check_status()
    worst = 0.0
    for (rid, p), row in got.items():
        ref = refs[rid][p]
        scale = float(refs[rid].abs().max())
        err = float((row - ref).abs().max()) / scale
        worst = max(worst, err)
        assert err <= bound, (rid, p, err)
        top = ref.topk(2).values
        if dtype == "float32" or float(top[0] - top[1]) > 2 * bound * scale:
            assert int(row.argmax()) == int(ref.argmax()), (rid, p)
    # the rows compared would show a lost page: with one page of sixteen keys hidden, the
    # plain logits themselves move by more than twice the bound at some of them
    scale = float(refs["long"].abs().max())
    moved = max(float((damaged[p] - refs["long"][p]).abs().max()) / scale
                for (rid, p) in got if rid == "long" and p >= 1040)
    assert moved > 2 * LONG_BOUNDS[1][1], moved
    print(f"long context {dtype}: worst relative error {worst:.2e} over {len(got)} rows "
          f"(a lost page would move them by {moved:.2f})")


def test_preemption_lookahead_and_portion_graphs_in_bfloat16(tmp_path_factory):
    """Generation through the entry point in bfloat16 at head size 64 (LFM2-350M widths, four
    layers): a pool so small that sequences are preempted and recomputed, prompt portions of
    one fixed size (their step shapes are captured and replayed), and the next decode step
    launched before the current one's tokens are read.  A recomputed sequence runs its
    generated tokens through the prompt kernels, so its logits differ from the unpreempted
    run's by bfloat16 rounding; every token must therefore be explained by the plain
    implementation's logits for the tokens before it (the plain winner, or within twice the
    bound of it), and where nothing was preempted the tokens equal those without lookahead."""
    from rvllm_b200 import GenerateOptions, Generator
    cfg = config_from_dict(LONG)
    folder = write_random_model(str(tmp_path_factory.mktemp("lfm2_gen")), cfg, 9)
    plain = PlainModel(folder)
    rng = random.Random(10)
    prompts = [[rng.randrange(4096) for _ in range(n)] for n in (200, 64, 129, 40, 300)]
    gen = Generator.load(folder, dtype="bfloat16")
    bound = BF16_BOUND_4_LAYERS

    def explained(outs):
        for p, o in zip(prompts, outs):
            ref = plain.logits(p + o)
            scale = float(ref.abs().max())
            for k, tok in enumerate(o):
                row = ref[len(p) + k - 1]
                assert float(row.max() - row[tok]) <= 2 * bound * scale, (len(p), k)

    roomy = GenerateOptions(max_tokens=40, block_size=16, stop_tokens=[], prefill_chunk=64)
    tight = GenerateOptions(max_tokens=40, block_size=16, stop_tokens=[], prefill_chunk=64,
                            num_blocks=40)               # 640 tokens for 733 + 5 x 40
    gen.lookahead = False
    plain_run = gen.complete_batch(prompts, roomy, arrival_steps=[0, 0, 1, 2, 4])
    explained(plain_run)
    gen.lookahead = True
    ahead = gen.complete_batch(prompts, roomy, arrival_steps=[0, 0, 1, 2, 4])
    assert ahead == plain_run
    runner = gen._runner
    assert runner.graph_steps > 0 and runner.capture_failures == 0
    assert len(runner._shape_graphs) + len(runner._mixed_graphs) > 0      # prompt portions replayed too
    squeezed = gen.complete_batch(prompts, tight, arrival_steps=[0, 0, 1, 2, 4])
    assert gen.last_result.stats.preemptions > 0
    assert all(len(o) == 40 for o in squeezed)
    explained(squeezed)
    gen.ops.check_status()
