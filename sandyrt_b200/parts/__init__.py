"""Parts a model is assembled from.  Importing this package registers the built-in kinds."""
from . import attention, block, mlp, norm, position  # noqa: F401
from .base import (Block, FeedForward, LayerCallCtx, Mixer, Norm, PagedKVSpec, Part,  # noqa: F401
                   PositionEncoding, StateSpec, StepContext, Workspace)
from .embedding import OutputHead, TokenEmbedding  # noqa: F401
from .linear import Linear  # noqa: F401
