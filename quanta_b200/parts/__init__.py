"""Parts a model is put together from; importing this package registers the built-in ones."""
from . import attention, block, moe, norms, rotary  # noqa: F401
from .base import (Block, FeedForward, KVCacheSpec, LayerCache, Mixer, Norm, Part, PositionEncoding,  # noqa: F401
                   StepContext, TensorSpec, make, register, registered)
from .spec import ModelSpec, ScheduleEntry  # noqa: F401
