"""Parts a model is put together from.  Importing the package registers the built-in
kinds; further kinds are added with `register_part` (see `base`)."""
from . import base
from .base import (Block, BuildContext, CacheNeed, FeedForward, KVNeed, LayerSpec, Mixer, ModelSpec, Norm, Part,
                   PartSpec, PendingSum, PositionEncoding, ScheduleEntry, StateNeed, StreamOp, WeightSpec, WeightStore, build_part,
                   known_parts, register_part)
from . import (attention, block, chunked_attention, embedding, latent_attention, mlp, moe, norm, reentry, rope,  # noqa: F401
               side_by_side, state_mixers)  # (registration)
from .linear import Linear
