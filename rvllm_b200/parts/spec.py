"""Descriptions of a model as data.

A model is a list of blocks; a block names an arrangement, a mixer, a feed-forward
and its norms; each of these is a small frozen record of sizes and constants.  The
order in which blocks run is a list of `LayerCall`s, so a block can run twice and a
call can read the cache that an earlier call wrote.  Nothing here knows which
architecture it describes: an architecture is a function from its configuration to a
`ModelSpec` (see `rvllm_b200.models`).

The reference expresses the same variability as one parameterised `Layer` with a
`Mixer` enum and optional tensors (src/model.rs:126-195).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class ParamDecl:
    """One tensor a part needs.

    shape      shape the part works with
    init       distribution of the random-weights mode, by name:
               "linear" and "embedding" N(0, 0.02), "conv" N(0, 0.2),
               "norm" 1 + N(0, 0.05), "bias" N(0, 0.02), "zeros";
               or "normal" with the part's own `mean` and `std`
    mean, std  given, they replace the named distribution's values, so a part outside
               this package can ask for any normal distribution
    alt_shapes shapes a file may store instead (same element count; reshaped on load)
    integer    an integer table: kept as int32 whatever the compute dtype
    """
    shape: Tuple[int, ...]
    init: str
    alt_shapes: Tuple[Tuple[int, ...], ...] = ()
    integer: bool = False
    mean: Optional[float] = None
    std: Optional[float] = None


@dataclass(frozen=True)
class NormSpec:
    kind: str
    size: int
    eps: float


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter the attention mixer. kind "none" applies nothing."""
    kind: str
    head_dim: int = 0
    theta: float = 0.0
    max_position: int = 0


@dataclass(frozen=True)
class MixerSpec:
    kind: str
    hidden: int


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: Optional[NormSpec] = None          # per-head norm of q and k before rotation
    position: PositionSpec = PositionSpec("none")
    window: Optional[int] = None                # keys visible: the last `window` positions
    scale: Optional[float] = None               # None: 1/sqrt(head_dim)
    # local tensor name -> suffix in the file
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class ShortConvSpec(MixerSpec):
    taps: int = 0                               # filter length; the state holds taps-1 rows
    bias: bool = False
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str
    hidden: int


@dataclass(frozen=True)
class SwiGLUSpec(FeedForwardSpec):
    ffn_dim: int = 0
    names: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which parts and how they are arranged.

    `norms` maps a place in the block to (norm spec, tensor name in the file); which
    places exist is the arrangement's business.  "pre_norm" (src/model.rs:556-585):
        h = x + post_mixer(mixer(mixer_norm(x)));  out = h + post_ffn(ffn(ffn_norm(h)))
    with places "mixer" and "ffn" required and "post_mixer", "post_ffn" optional (the
    reference's `post_attn_norm` and `post_ffn_norm`, src/model.rs:571, 581; LFM2 has
    neither).  The *_prefix fields say where the mixer's and the feed-forward's tensors
    are found in the file.
    """
    arrangement: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    norms: Mapping[str, Tuple[NormSpec, str]] = field(hash=False)
    mixer_prefix: str = ""
    ffn_prefix: str = ""


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block `layer`; `cache_of`, if given, is the
    index (in the order list) of an earlier call whose cache this call reads instead of
    owning one."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    max_position: int
    layers: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: str
    head_name: Optional[str]                    # None: the head is the embedding table
    embedding_scale: Optional[float] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
