"""Parts a decoder is assembled from.  Importing the package registers the built-in kinds."""

from .base import (Block, FeedForward, LayerCall, LayerSpec, Mixer, ModelPlan, Norm, NormedUpdate, Part, PartSpec,
                   PositionEncoding, ScaledUpdate, StreamCall, StreamOp, WeightSpec, build_part, register_part, registered,
                   settle_update)
from . import (attention, block, delta, diff_attention, embedding, glu, latent_attention, layernorm, mlp, moe,  # noqa: F401
               reentry, rmsnorm, rope, ssd, swiglu)                                                                       # (registration)

__all__ = ["Block", "FeedForward", "LayerCall", "LayerSpec", "Mixer", "ModelPlan", "Norm", "NormedUpdate", "Part",
           "PartSpec", "PositionEncoding", "ScaledUpdate", "StreamCall", "StreamOp", "WeightSpec", "build_part", "register_part",
           "registered", "settle_update"]
