"""Parts that layers are put together from. Importing the package registers them."""
from . import (attention, attention_mixed, attention_sink, block, feed_forward,  # noqa: F401
               norm, parallel, position, retention, state_space)
from .base import CacheNeed, LayerCache, Part, StateNeed, StepContext  # noqa: F401
