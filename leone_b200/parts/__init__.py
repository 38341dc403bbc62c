"""Parts a layer is built from.  Importing this package registers the built-in kinds."""
from . import (attention, block, embedding, experts, gated_delta, head, injection, latent_attention,  # noqa: F401
               linear_attention, min_gru, mlp, pooled_attention, rms_norm, rotary, short_conv, side_by_side, swiglu,
               token_gate)
from .base import (Block, Embedding, FeedForward, FixedState, Head, Mixer, Norm, PagedCacheView, PagedKV, Part,
                   PositionEncoding, Runtime, StateView, WeightSpec)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["Block", "Embedding", "FeedForward", "FixedState", "Head", "Mixer", "Norm", "PagedCacheView", "PagedKV",
           "Part", "PositionEncoding", "Runtime", "StateView", "WeightSpec", "LayerSpec",
           "ModelSpec", "PartSpec"]
