from . import standard  # registers the standard parts
from .base import (CacheRequest, Embedding, FeedForward, Head, Mixer, Norm, Part,
                   PositionEncoding, TensorRequest, build_part, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm,
                   register_position, registered)
from .model import Block, CacheGroup, Model, PreNormBlock, register_arrangement
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

__all__ = [
    "Block", "CacheGroup", "CacheRequest", "Embedding", "FeedForward", "Head", "LayerCall",
    "LayerSpec", "Mixer", "Model", "ModelSpec", "Norm", "Part", "PartSpec", "PositionEncoding",
    "PreNormBlock", "TensorRequest", "build_part", "register_arrangement",
    "register_embedding", "register_feed_forward", "register_head", "register_mixer",
    "register_norm", "register_position", "registered",
]
