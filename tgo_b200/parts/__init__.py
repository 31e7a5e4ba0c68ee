"""Parts that layers are put together from. Importing the package registers them."""
from . import (attention, attention_latent, attention_mixed, attention_sink, block,  # noqa: F401
               feed_forward, mlstm, norm, parallel, position, retention, state_space)
from .base import CacheNeed, LayerCache, Part, StateNeed, StepContext  # noqa: F401
