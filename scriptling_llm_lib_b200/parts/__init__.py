from . import (attention, block, delta_rule, embedding, experts, feedforward, latent_attention, linear_attention, norm, parallel, pass_vector, rglru,
               rotary, selective_scan, token_side)  # noqa: F401  (registers the built-in parts)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, STREAM_INPUTS, Embedding, FeedForward,
                   Head, Mixer, Norm, Part, PartSpec, PositionEncoding, StreamInput)
from .block import Block, LayerSpec, build_block, pre_norm_layer
from .embedding import OutputHead, TokenEmbedding, linear_head, token_embedding
from .linear import Linear

__all__ = ["ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "STREAM_INPUTS", "StreamInput", "Embedding",
           "FeedForward", "Head", "Mixer", "Norm", "Part", "PartSpec", "PositionEncoding", "Block", "LayerSpec", "build_block",
           "pre_norm_layer", "OutputHead", "TokenEmbedding", "linear_head", "token_embedding", "Linear"]
