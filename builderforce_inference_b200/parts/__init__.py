"""Parts a decoder is put together from.  Importing this package registers the built-in kinds."""
from .base import (BLOCKS, FEED_FORWARDS, INPUT_PARTS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, InputPart, KVNeed,
                   LayerSpec, Mixer, ModelSpec, Norm, ParamSpec, Part, PartSpec, PositionEncoding, Registry,
                   RunSpec, StateNeed)
from . import attention, block, combine, inputs, latent, lightning, mlp, moe, norm, recurrent, rotary  # noqa: F401  (registration)

__all__ = ["BLOCKS", "FEED_FORWARDS", "INPUT_PARTS", "InputPart", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "FeedForward",
           "KVNeed", "LayerSpec", "Mixer", "ModelSpec", "Norm", "ParamSpec", "Part", "PartSpec",
           "PositionEncoding", "Registry", "RunSpec", "StateNeed"]
