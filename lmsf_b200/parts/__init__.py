"""Parts of a model and their registries.  Importing this package registers the built-in kinds."""
from .base import (Block, CacheGroupView, FeedForward, KVCacheSpec, LayerCache, LayerCall, LayerSpec, Mixer, ModelSpec,
                   Norm, Part, PartSpec, PositionEncoding, Shift, StateSpec, StepContext, WeightSpec, build_part, part_class,
                   register_part)
from . import (attention, block, embedding, latent_attention, lightning, linear, mlp, moe, norm, recurrent, rope,  # noqa: F401
               shift, stream_entry, token_gate)  # (registration)
