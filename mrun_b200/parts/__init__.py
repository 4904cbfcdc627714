"""Parts a layer is assembled from.  Importing the package registers the built-in kinds."""
from . import attention, block, feedforward, norm, rotary  # noqa: F401  (registration)
from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, TRANSFORMS, Precision, Runtime,
                   register_arrangement, register_feed_forward, register_mixer, register_norm,
                   register_position, register_transform)

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "TRANSFORMS", "Precision", "Runtime",
           "register_arrangement", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "register_transform"]
