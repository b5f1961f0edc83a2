"""LFM2 (`Lfm2ForCausalLM`): from its configuration to a `ModelSpec`.

Layer i is an attention block when i is in `full_attn_idxs`, else a gated
short-convolution block (the reference derives the same from the per-layer KV-head
array, 0 meaning a convolution layer, src/weights.rs:159-178).  Every block is
pre-norm with a SwiGLU feed-forward; q and k are RMS-normalised per head before the
rotation; no biases except the optional convolution biases; no post-norms; the final
norm is the checkpoint's `embedding_norm` (src/weights.rs:105-148).

Tensor names are those of the architecture's safetensors checkpoints; the reference's
GGUF names (src/weights.rs:365-433) map to them as
  token_embd -> model.embed_tokens            token_embd_norm -> model.embedding_norm
  blk.i.attn_norm -> layers.i.operator_norm   blk.i.ffn_norm -> layers.i.ffn_norm
  blk.i.shortconv.{in_proj,conv,out_proj} -> layers.i.conv.{in_proj,conv,out_proj}
  blk.i.attn_{q,k,v,output} -> layers.i.self_attn.{q,k,v,out}_proj
  blk.i.attn_{q,k}_norm -> layers.i.self_attn.{q,k}_layernorm
  blk.i.ffn_{gate,up,down} -> layers.i.feed_forward.{w1,w3,w2}
"""
from __future__ import annotations

from ..config.lfm2 import ATTENTION, Lfm2Config
from ..config.registry import register_architecture
from ..parts.spec import (AttentionSpec, BlockSpec, LayerCall, ModelSpec, NormSpec,
                          PositionSpec, ShortConvSpec, SwiGLUSpec)

_ATTN_NAMES = {"q_norm": "q_layernorm.weight", "k_norm": "k_layernorm.weight"}
_FFN_NAMES = {"gate": "w1.weight", "up": "w3.weight", "down": "w2.weight"}


def build_spec(cfg: Lfm2Config) -> ModelSpec:
    hidden = cfg.hidden_size
    norm = NormSpec("rmsnorm", hidden, cfg.norm_eps)
    ffn = SwiGLUSpec("swiglu", hidden, ffn_dim=cfg.ffn_dim, names=_FFN_NAMES)
    attention = AttentionSpec(
        "attention", hidden,
        num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim,
        qk_norm=NormSpec("rmsnorm", cfg.head_dim, cfg.norm_eps),
        position=PositionSpec("rope", cfg.head_dim, cfg.rope_theta,
                              cfg.max_position_embeddings),
        window=None, scale=None, names=_ATTN_NAMES)
    conv = ShortConvSpec("short_conv", hidden, taps=cfg.conv_L_cache, bias=cfg.conv_bias)
    layers = []
    for i, kind in enumerate(cfg.layer_kinds):
        p = f"model.layers.{i}."
        is_attn = kind == ATTENTION
        layers.append(BlockSpec(
            arrangement="pre_norm",
            mixer=attention if is_attn else conv,
            feed_forward=ffn,
            norms={"mixer": (norm, p + "operator_norm.weight"),
                   "ffn": (norm, p + "ffn_norm.weight")},
            mixer_prefix=p + ("self_attn." if is_attn else "conv."),
            ffn_prefix=p + "feed_forward."))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden=hidden,
        max_position=cfg.max_position_embeddings, layers=tuple(layers),
        order=tuple(LayerCall(i) for i in range(len(layers))),
        final_norm=norm, embedding_name="model.embed_tokens.weight",
        final_norm_name="model.embedding_norm.weight",
        head_name=None if cfg.tie_embedding else "lm_head.weight",
        bos_token_id=cfg.bos_token_id, eos_token_id=cfg.eos_token_id)


register_architecture("Lfm2ForCausalLM", Lfm2Config, build_spec, replace=True)
