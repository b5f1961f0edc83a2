"""The tiny configurations the tests use, and helpers to write them as model folders.

TINY_A and TINY_B differ in every size and option: layer count and kinds, hidden
width, head counts and group size, head size, feed-forward rule, filter length and
bias, vocabulary, rotation base, context, norm eps, tied or untied head.
"""
import copy
import os

from rvllm_b200.config import config_from_dict
from rvllm_b200.weights import write_random_model

TINY_A = {
    "architectures": ["Lfm2ForCausalLM"],
    "num_hidden_layers": 4, "full_attn_idxs": [1, 3],
    "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "block_ff_dim": 192, "block_auto_adjust_ff_dim": False,
    "conv_L_cache": 3, "conv_bias": False,
    "vocab_size": 512, "rope_theta": 1000000.0, "max_position_embeddings": 256,
    "norm_eps": 1e-5, "tie_embedding": True, "torch_dtype": "bfloat16",
    "bos_token_id": 1, "eos_token_id": 7,
}

TINY_B = {
    "architectures": ["Lfm2ForCausalLM"],
    "num_hidden_layers": 6, "full_attn_idxs": [2, 5],
    "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "block_ff_dim": 384, "block_auto_adjust_ff_dim": True, "block_multiple_of": 128,
    "conv_L_cache": 4, "conv_bias": True,
    "vocab_size": 1000, "rope_theta": 10000.0, "max_position_embeddings": 512,
    "norm_eps": 1e-6, "tie_embedding": False, "torch_dtype": "bfloat16",
    "bos_token_id": 1, "eos_token_id": 2,
}

SEEDS = {"A": 0, "B": 1}


def tiny(name: str) -> dict:
    return copy.deepcopy({"A": TINY_A, "B": TINY_B}[name])


def write_tiny(folder: str, name: str, **overrides) -> str:
    data = tiny(name)
    data.update(overrides)
    cfg = config_from_dict(data)
    return write_random_model(os.path.join(folder, "tiny_" + name), cfg, SEEDS[name])
