"""Greedy and seeded generation through the entry points on the GPU."""
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import schedules
from plain_lfm2 import PlainModel
from plain_ops import sample_row
from tiny import write_tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {n: write_tiny(root, n) for n in ("A", "B")}


def test_greedy_tiny_a_workload(folders):
    """Tiny A's workload: prompts of 5, 17 and 31 tokens, 16 new tokens each, pages of 8;
    float32 tokens equal the plain implementation's under every scheduling."""
    from rvllm_b200 import GenerateOptions, Generator
    plain = PlainModel(folders["A"])
    rng = random.Random(0)
    prompts = [[rng.randrange(512) for _ in range(n)] for n in (5, 17, 31)]
    want = [plain.greedy(p, 16) for p in prompts]
    gen = Generator.load(folders["A"], dtype="float32")
    for opts in (GenerateOptions(max_tokens=16, block_size=8, stop_tokens=[]),
                 GenerateOptions(max_tokens=16, block_size=8, stop_tokens=[], prefill_chunk=4,
                                 max_batched_tokens=9),
                 GenerateOptions(max_tokens=16, block_size=8, stop_tokens=[], num_blocks=9,
                                 prefill_chunk=6)):
        assert gen.complete_batch(prompts, opts) == want
    assert gen.last_result.stats.preemptions > 0
    assert gen.complete(prompts[1], GenerateOptions(max_tokens=16, block_size=8,
                                                    stop_tokens=[])) == want[1]


def test_generator_keeps_its_pool_between_calls(folders):
    """A pool sized for a call's own requests is used again by a later call that fits into it
    (no new cache, no new captures); a larger call grows it; a pool the caller asks for by
    size is made exactly; the tokens are the plain implementation's every time."""
    from rvllm_b200 import GenerateOptions, Generator
    plain = PlainModel(folders["A"])
    rng = random.Random(3)
    prompts = [[rng.randrange(512) for _ in range(n)] for n in (40, 9, 23, 60)]
    want = [plain.greedy(p, 8) for p in prompts]
    gen = Generator.load(folders["A"], dtype="float32")
    opts = GenerateOptions(max_tokens=8, block_size=8, stop_tokens=[])
    assert gen.complete(prompts[3], opts) == want[3]            # 9 pages of 8
    first = gen._runner
    assert gen.complete(prompts[1], opts) == want[1] and gen._runner is first
    assert gen.complete_batch(prompts[1:3], opts) == want[1:3] and gen._runner is first   # 7 pages
    assert gen.complete_batch(prompts, opts) == want            # 22 pages: a new pool
    grown = gen._runner
    assert grown is not first and grown.cache.num_pages >= 22
    assert gen.complete(prompts[3], opts) == want[3] and gen._runner is grown
    exact = GenerateOptions(max_tokens=8, block_size=8, stop_tokens=[], num_blocks=11)
    assert gen.complete(prompts[2], exact) == want[2]
    assert gen._runner.cache.num_pages == 11


def test_random_workloads_equal_plain(folders):
    """Rounds of three to eight requests with random prompt lengths, arrival steps, portion
    sizes, token budgets and pool sizes (some so small that sequences are preempted), all
    through one generator, so that pools, captured single-token steps and captured padded
    mixtures are used again from round to round: float32 greedy tokens equal the plain
    implementation's every time."""
    from rvllm_b200 import GenerateOptions, Generator
    plain = PlainModel(folders["B"])
    gen = Generator.load(folders["B"], dtype="float32")
    rng = random.Random(7)
    preempted = replayed = 0
    for _ in range(8):
        n = rng.randrange(3, 9)
        prompts = [[rng.randrange(900) for _ in range(rng.randrange(3, 140))] for _ in range(n)]
        arrivals = sorted(rng.randrange(0, 12) for _ in range(n))
        opts = GenerateOptions(max_tokens=rng.randrange(4, 30), block_size=16, stop_tokens=[],
                               prefill_chunk=rng.choice([None, 16, 37, 64]),
                               max_batched_tokens=rng.choice([48, 96, 8192]),
                               num_blocks=rng.choice([None, None, 14, 20]))
        outs = gen.complete_batch(prompts, opts, arrival_steps=arrivals)
        assert outs == [plain.greedy(p, opts.max_tokens) for p in prompts]
        preempted += gen.last_result.stats.preemptions
        replayed += len(gen._runner._mixed_graphs)
        assert gen._runner.capture_failures == 0
    assert preempted > 0 and replayed > 0


def test_stop_token_ends_and_is_stripped(folders):
    from rvllm_b200 import GenerateOptions, Generator
    plain = PlainModel(folders["A"])
    prompt = [9, 8, 7, 6, 5]
    free = plain.greedy(prompt, 10)
    gen = Generator.load(folders["A"], dtype="float32")
    got = gen.complete(prompt, GenerateOptions(max_tokens=10, stop_tokens=[free[4]]))
    first = free.index(free[4])
    assert got == free[:first]


def test_seeded_temperature_tiny_b_workload(folders):
    """Tiny B's workload: 5 requests, arrivals 0/0/2/5/7, temperature 0.8 seeded, 24 new
    tokens, pages of 16, portions of 32.  Checked by teacher forcing: the sampled tokens
    are fed to the plain implementation and every token must be the one the sampler's
    definition picks from the plain logits (or, where float32 rounding moves a draw across
    a boundary, the engine's own logits must explain it)."""
    from rvllm_b200 import GenerateOptions, Generator
    plain = PlainModel(folders["B"])
    rng = random.Random(1)
    prompts = [[rng.randrange(1000) for _ in range(n)] for n in (1, 9, 40, 64, 100)]
    gen = Generator.load(folders["B"], dtype="float32")
    opts = GenerateOptions(max_tokens=24, temperature=0.8, seed=11, block_size=16,
                           prefill_chunk=32, stop_tokens=[])
    outs = gen.complete_batch(prompts, opts, arrival_steps=[0, 0, 2, 5, 7])
    again = gen.complete_batch(prompts, opts, arrival_steps=[0, 0, 0, 0, 0])
    assert outs == again                     # a seeded request does not depend on its batch
    differ = 0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o) == 24
        logits = plain.logits(p + o)
        for k, tok in enumerate(o):
            want = sample_row(logits[len(p) + k - 1], 0.8, 1.0, 11 + i, k)
            differ += int(want != tok)
    assert differ <= 1


def test_cli_prints_one_completion_per_prompt(folders):
    plain = PlainModel(folders["A"])
    p1, p2 = [3, 1, 4, 1, 5, 9, 2, 6], [2, 7, 1, 8]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "rvllm"), "cli", "--model", folders["A"],
           "--dtype", "float32", "--token-ids", "--prompt", " ".join(map(str, p1)),
           "--prompt", ",".join(map(str, p2)), "--max-tokens", "6", "--arrival-step", "0",
           "--arrival-step", "3", "--block-size", "8"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.strip().splitlines() if l.strip()]
    eos = 7

    def strip(toks):
        return toks[:toks.index(eos)] if eos in toks else toks
    assert [int(t) for t in lines[0].split()] == strip(plain.greedy(p1, 6))
    assert [int(t) for t in lines[1].split()] == strip(plain.greedy(p2, 6))


def test_trace_run_program(folders, tmp_path):
    """bin/trace_run as a user runs it: steps on stdin, `done` lines, .f32 files."""
    plain = PlainModel(folders["B"])
    rng = random.Random(4)
    reqs = {f"q{i}": [rng.randrange(1000) for _ in range(n)] for i, n in enumerate((70, 33, 90, 41, 12))}
    steps = schedules.mixed(reqs, seed=2)
    import json
    for dtype, bound in (("float32", 1e-5), ("bfloat16", 3e-2)):
        out = tmp_path / dtype
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"],
               "--dtype", dtype, "--out", str(out), "--max-tokens",
               str(schedules.tokens_held(steps, 64))]
        r = subprocess.run(cmd, input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.split("\n") if l.startswith("done")] == \
            [f"done {s['step']}" for s in steps]
        pos = {k: 0 for k in reqs}
        refs = {k: plain.logits(v) for k, v in reqs.items()}
        for s in steps:
            arr = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, 1000)
            k = 0
            for e in s["entries"]:
                for w in e["want"]:
                    ref = refs[e["id"]][pos[e["id"]] + w]
                    err = float((torch.from_numpy(arr[k].copy()) - ref).abs().max() / ref.abs().max())
                    assert err <= bound, (dtype, s["step"], e["id"], w, err)
                    k += 1
                pos[e["id"]] += len(e["tokens"])
            assert k == arr.shape[0]


def test_lookahead_gives_the_same_tokens(folders):
    """Launching the next decode step before the current one's tokens are read changes
    nothing a request sees: stop tokens in the middle, requests of different lengths,
    a pool that forces preemption, and seeded sampling."""
    from rvllm_b200 import GenerateOptions, Generator
    rng = random.Random(6)
    prompts = [[rng.randrange(512) for _ in range(n)] for n in (3, 20, 9, 33)]
    gen = Generator.load(folders["A"], dtype="float32")
    cases = [GenerateOptions(max_tokens=30, block_size=8, stop_tokens=[]),
             GenerateOptions(max_tokens=30, block_size=8, stop_tokens=[97, 5, 300]),
             GenerateOptions(max_tokens=25, block_size=8, stop_tokens=[], num_blocks=14),
             GenerateOptions(max_tokens=30, block_size=8, temperature=0.9, top_p=0.8, seed=3)]
    for opts in cases:
        gen.lookahead = False
        want = gen.complete_batch(prompts, opts, arrival_steps=[0, 0, 3, 4])
        gen.lookahead = True
        got = gen.complete_batch(prompts, opts, arrival_steps=[0, 0, 3, 4])
        assert got == want
