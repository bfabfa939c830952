"""Parts of a layer.  Importing this package registers the built-in parts."""
from . import attention, block, ffn, norm, rope  # noqa: F401
from .base import BuildContext, FeedForward, Mixer, Norm, Part, PositionEncoding  # noqa: F401
