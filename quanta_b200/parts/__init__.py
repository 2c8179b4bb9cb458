"""Parts a model is put together from; importing this package registers the built-in ones."""
from . import attention, block, moe, norms, rotary  # noqa: F401
from .base import (Block, CacheSpec, CacheStream, Embedding, FeedForward, Head, KeepAll, KVCacheSpec,  # noqa: F401
                   LayerCache, Mixer, Norm, Part, PositionEncoding, Retention, StepContext, TensorSpec, Window, make,
                   register, registered)
from .spec import ModelSpec, ScheduleEntry  # noqa: F401
