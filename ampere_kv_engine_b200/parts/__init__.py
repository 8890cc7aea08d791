"""The parts a model is put together from.  Importing the package registers the built-in kinds."""

from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401
