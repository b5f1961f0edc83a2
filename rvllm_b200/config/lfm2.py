"""The LFM2 configuration: gated short-convolution layers beside grouped-query
attention layers.

The reference reads the same quantities from GGUF metadata
(`Config::from_gguf_metadata`, src/weights.rs:152-293); here they come from the
architecture's config.json keys.  Every size is read from the file; the few keys
with a default are options whose absence has one meaning (no bias, no multiplier,
tied embeddings, head size = hidden / heads as at src/weights.rs:195-201).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .base import Reader

CONV = "conv"
ATTENTION = "full_attention"


@dataclass(frozen=True)
class Lfm2Config:
    architecture: str
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    norm_eps: float
    rope_theta: float
    full_attn_idxs: Tuple[int, ...]
    conv_L_cache: int
    conv_bias: bool
    block_ff_dim: int
    block_auto_adjust_ff_dim: bool
    block_multiple_of: Optional[int]
    block_ffn_dim_multiplier: Optional[float]
    tie_embedding: bool
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    # ---- derived -----------------------------------------------------------------

    @property
    def ffn_dim(self) -> int:
        """Width of the SwiGLU hidden layer after the adjustment rule.

        The reference reads the adjusted number (src/weights.rs:276); config.json
        carries the unadjusted one and the rule: two thirds, times the optional
        multiplier, rounded up to `block_multiple_of`.
        """
        f = self.block_ff_dim
        if self.block_auto_adjust_ff_dim:
            f = int(2 * f / 3)
            if self.block_ffn_dim_multiplier is not None:
                f = int(self.block_ffn_dim_multiplier * f)
            m = self.block_multiple_of
            f = m * ((f + m - 1) // m)
        return f

    @property
    def layer_kinds(self) -> List[str]:
        attn = set(self.full_attn_idxs)
        return [ATTENTION if i in attn else CONV for i in range(self.num_hidden_layers)]

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ---- reading -----------------------------------------------------------------

    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "Lfm2Config":
        r = Reader(data, where)
        archs = r.str_list("architectures")
        if not archs:
            raise ConfigError(f"{where}: key 'architectures' is empty")
        layers = r.int("num_hidden_layers", minimum=1)
        hidden = r.int("hidden_size", minimum=1)
        heads = r.int("num_attention_heads", minimum=1)
        kv_heads = r.int("num_key_value_heads", minimum=1)
        # Grouped-query attention shares each KV head with a whole group of query
        # heads (src/weights.rs:188-192).
        if heads % kv_heads != 0:
            raise ConfigError(
                f"{where}: invalid attention head counts: {heads} query, {kv_heads} KV")
        if r.has("head_dim"):
            head_dim = r.int("head_dim", minimum=1)
        elif hidden % heads == 0:
            head_dim = hidden // heads
        else:
            raise ConfigError(
                f"{where}: no 'head_dim' and hidden_size {hidden} isn't divisible by {heads} heads")
        # The rotation pairs dimension i with i + head_dim/2 (src/weights.rs:203-206).
        if head_dim % 2 != 0:
            raise ConfigError(f"{where}: invalid attention head size {head_dim}: must be even")

        if r.has("full_attn_idxs"):
            attn = r.int_list("full_attn_idxs")
        elif r.has("layer_types"):
            kinds = r.str_list("layer_types")
            if len(kinds) != layers:
                raise ConfigError(
                    f"{where}: 'layer_types' has {len(kinds)} entries for {layers} layers")
            bad = sorted(set(kinds) - {CONV, ATTENTION})
            if bad:
                raise ConfigError(f"{where}: unknown layer types {bad} "
                                  f"(known: {CONV!r}, {ATTENTION!r})")
            attn = [i for i, k in enumerate(kinds) if k == ATTENTION]
        else:
            raise ConfigError(f"{where}: missing key 'full_attn_idxs' (or 'layer_types')")
        if any(i < 0 or i >= layers for i in attn):
            raise ConfigError(f"{where}: 'full_attn_idxs' {attn} out of range for {layers} layers")
        if sorted(set(attn)) != attn:
            raise ConfigError(f"{where}: 'full_attn_idxs' {attn} must be sorted and unique")
        if not attn:
            # src/weights.rs:182-184
            raise ConfigError(f"{where}: no attention layers")

        n_conv = layers - len(attn)
        taps = r.int("conv_L_cache", minimum=1) if (n_conv or r.has("conv_L_cache")) else 1
        auto = r.bool("block_auto_adjust_ff_dim")
        multiple = r.optional_int("block_multiple_of", minimum=1)
        if auto and multiple is None:
            raise ConfigError(f"{where}: 'block_auto_adjust_ff_dim' is on but "
                              f"'block_multiple_of' is missing")
        if r.has("tie_embedding"):
            tie = r.bool("tie_embedding")
        elif r.has("tie_word_embeddings"):
            tie = r.bool("tie_word_embeddings")
        else:
            tie = True
        known = {
            "architectures", "num_hidden_layers", "hidden_size", "num_attention_heads",
            "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings",
            "norm_eps", "rope_theta", "full_attn_idxs", "layer_types", "conv_L_cache",
            "conv_bias", "block_ff_dim", "block_auto_adjust_ff_dim", "block_multiple_of",
            "block_ffn_dim_multiplier", "tie_embedding", "tie_word_embeddings",
            "bos_token_id", "eos_token_id", "torch_dtype",
        }
        return cls(
            architecture=archs[0],
            num_hidden_layers=layers,
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=r.int("vocab_size", minimum=1),
            max_position_embeddings=r.int("max_position_embeddings", minimum=1),
            norm_eps=r.float("norm_eps"),
            rope_theta=r.float("rope_theta"),
            full_attn_idxs=tuple(attn),
            conv_L_cache=taps,
            conv_bias=r.bool("conv_bias", False),
            block_ff_dim=r.int("block_ff_dim", minimum=1),
            block_auto_adjust_ff_dim=auto,
            block_multiple_of=multiple,
            block_ffn_dim_multiplier=r.optional_float("block_ffn_dim_multiplier"),
            tie_embedding=tie,
            bos_token_id=r.optional_int("bos_token_id"),
            eos_token_id=r.optional_int("eos_token_id"),
            torch_dtype=r.str("torch_dtype", "bfloat16"),
            extra={k: v for k, v in data.items() if k not in known},
        )

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        d.update(
            architectures=[self.architecture],
            num_hidden_layers=self.num_hidden_layers,
            hidden_size=self.hidden_size,
            num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads,
            head_dim=self.head_dim,
            vocab_size=self.vocab_size,
            max_position_embeddings=self.max_position_embeddings,
            norm_eps=self.norm_eps,
            rope_theta=self.rope_theta,
            full_attn_idxs=list(self.full_attn_idxs),
            layer_types=self.layer_kinds,
            conv_L_cache=self.conv_L_cache,
            conv_bias=self.conv_bias,
            block_ff_dim=self.block_ff_dim,
            block_auto_adjust_ff_dim=self.block_auto_adjust_ff_dim,
            tie_embedding=self.tie_embedding,
            torch_dtype=self.torch_dtype,
        )
        for key in ("block_multiple_of", "block_ffn_dim_multiplier", "bos_token_id",
                    "eos_token_id"):
            if getattr(self, key) is not None:
                d[key] = getattr(self, key)
        return d
