from .spec import PartSpec, SubLayer, LayerSpec, ScheduleEntry, ModelSpec, BuildEnv  # noqa: F401
from .registry import (register_mixer, register_feed_forward, register_norm,  # noqa: F401
                       register_position_encoding, register_arrangement, register_embedding, register_head)
from .base import (Part, Mixer, FeedForward, Norm, PositionEncoding, Embedding, Head,  # noqa: F401
                   Arrangement, CacheView, Stream)
# the built-in parts register themselves on import
from . import attention, block, embedding, mlp, norm, rope  # noqa: E402,F401
