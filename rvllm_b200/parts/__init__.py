"""Parts a model is put together from: mixers, feed-forwards, norms, position
encodings and their arrangement in a block.  Importing the package registers the
built-in kinds."""
from . import attention, block, feed_forward, norm, position, short_conv  # noqa: F401
from .base import (Arrangement, FeedForward, Mixer, Norm, PagedNeed, PositionEncoding,
                   StateNeed, Stream, arrangement_class, feed_forward_class, mixer_class,
                   norm_class, position_class, register_arrangement,
                   register_feed_forward, register_mixer, register_norm,
                   register_position)
from .spec import (AttentionSpec, BlockSpec, FeedForwardSpec, LayerCall, MixerSpec,
                   ModelSpec, NormSpec, ParamDecl, PositionSpec, ShortConvSpec, SwiGLUSpec)
