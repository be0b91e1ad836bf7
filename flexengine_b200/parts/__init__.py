from . import attention, block, embedding, feed_forward, head, norm, position  # noqa: F401  (register the built-in kinds)
from .base import (Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, build_part, register_block,
                   register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                   register_position)
from .model import DecoderModel
from .spec import (CacheGroupSpec, LayerSpec, ModelPlan, PartSpec, RunEntry, WeightBinding, WeightSource)

__all__ = ["Embedding", "Head", "register_embedding", "register_head", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "build_part", "register_block",
           "register_feed_forward", "register_mixer", "register_norm", "register_position", "DecoderModel",
           "CacheGroupSpec", "LayerSpec", "ModelPlan", "PartSpec", "RunEntry", "WeightBinding", "WeightSource"]
