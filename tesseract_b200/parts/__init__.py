"""Parts of a decoder and their registries; importing this package registers the built-in kinds."""

from .base import (BLOCKS, DeferredNorm, EMBEDDINGS, FEED_FORWARDS, HEADS, INJECTIONS, Injection, MIXERS, NORMS, POSITION_ENCODINGS, Block,
                   CacheBinding, Embedding, FeedForward, FollowNorm, GroupView, Head, Mixer, Norm, PagedKeyValueNeed, PagedKVNeed, PagedNeed, PagedVectorNeed, Part, PooledBlocksNeed, PreparedNorm,
                   PositionEncoding, Registry, RESIDUAL_GATES, ResidualGates, ResidualStream, Runtime, StateNeed, StepContext, TOKEN_INPUTS, TokenInput)
from . import (attention, block, conv_attention, differential_attention, embedding, experts, injection, latent_attention,  # noqa: F401
               lightning, mlp, norm, normed_attention, parallel_mixers, recurrent, residual_gate, rotary, token_input)  # noqa: F401  (registration)
from .linear import Linear
