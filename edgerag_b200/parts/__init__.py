"""Parts a decoder is assembled from.  Importing the package registers the built-in kinds."""

from .base import (Block, FeedForward, LayerCall, LayerSpec, Mixer, ModelPlan, Norm, NormedUpdate, Part, PartSpec,
                   PositionEncoding, StreamCall, StreamOp, WeightSpec, build_part, register_part, registered,
                   settle_update)
from . import (attention, block, delta, embedding, glu, latent_attention, layernorm, moe, reentry, rmsnorm, rope,  # noqa: F401
               ssd, swiglu)                                                                       # (registration)

__all__ = ["Block", "FeedForward", "LayerCall", "LayerSpec", "Mixer", "ModelPlan", "Norm", "NormedUpdate", "Part",
           "PartSpec", "PositionEncoding", "StreamCall", "StreamOp", "WeightSpec", "build_part", "register_part",
           "registered", "settle_update"]
