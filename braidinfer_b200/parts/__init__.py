"""Parts that layers are made of.  Importing the package registers the built-in parts."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, INJECTIONS, LAYER_INPUTS, MIXERS, NORMS, POSITION_ENCODINGS,
                   Block, Embedding, FeedForward, Head, Injection, LayerInput, Mixer, Norm, Part, PositionEncoding,
                   Registry)
from .spec import CacheRequest, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
from .runtime import Runtime
from . import (attention, block, embedding, feedforward, injection, latent_attention, linear_attention,  # noqa: F401
               mlstm, moe, norm, parallel, rope, ssm, token_input)                                       # (registration)
