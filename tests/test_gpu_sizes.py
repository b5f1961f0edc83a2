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
            runner.step([StepEntry("r", ids[:-1], ())])
            before = ops.launches
            out[mode] = runner.step([StepEntry("r", ids[-1:], (0,))])[0].float().cpu()
            launches[mode] = ops.launches - before
    finally:
        ops.fuse_qkv_rope = fused
    ops.check_status()
    assert launches[False] - launches[True] == len(LFM2_350M["full_attn_idxs"])
    scale = float(out[False].abs().max())
    assert float((out[True] - out[False]).abs().max()) <= BF16_BOUND_16_LAYERS * scale
