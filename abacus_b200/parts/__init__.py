from .base import BLOCKS, FEED_FORWARDS, FRAMES, MIXERS, NORMS, POSITIONS, BuildContext, Registry
from .workspace import Workspace
from .linear import Linear
from . import attention, block, frame, mlp, norm, position  # noqa: F401  (register the built-in parts)

__all__ = ["BLOCKS", "FEED_FORWARDS", "FRAMES", "MIXERS", "NORMS", "POSITIONS", "BuildContext", "Registry", "Workspace", "Linear"]
