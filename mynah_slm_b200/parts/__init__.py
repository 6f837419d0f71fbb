"""Parts a layer is put together from. Importing the package registers the
built-in ones."""
from .base import (Block, CacheView, Embedding, FeedForward, Head, KVRequest, Mixer, Norm, Part, PositionEncoding,
                   Residual, StateRequest, TensorSpec, build_part, known_parts, register_block,
                   register_embedding, register_ffn, register_head, register_mixer, register_norm,
                   register_position)
from . import (attention, attention_capped, attention_latent, attention_projnorm, attention_sink, block, block_postnorm,  # noqa: F401
               block_sandwich, delta, embedding, feedforward, feedforward_dense, feedforward_routed,  # (registration)
               mamba, norms, norms_layer, parallel, position, recurrent_lru, retention)
from .embedding import LinearHead, TokenEmbedding
