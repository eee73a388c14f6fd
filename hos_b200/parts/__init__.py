"""The parts a layer is put together from.  Importing this package registers them."""
from . import attention, block, embedding, feedforward, norm, rope  # noqa: F401
