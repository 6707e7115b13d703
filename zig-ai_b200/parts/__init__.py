"""Parts that layers are put together from: mixers, feed-forwards, norms, position encodings and
the block that arranges them.  Importing this package registers the built-in parts."""
from .base import (Block, Embedding, FeedForward, Head, LazyNorm, Residual, LayerCall, LayerSpec, Mixer, ModelSpec, Norm,
                   PagedKVNeed, PagedRowsNeed, ParamDecl, Part, PartSpec, PositionEncoding, StateNeed, make_block,
                   make_part, needs_of, register_part, unregister_part)
from . import norms, position, feed_forward, short_conv, attention, block, embedding  # noqa: F401  (registration)
