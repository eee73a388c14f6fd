"""Architectures.  Importing this package registers them."""
from . import gemma2  # noqa: F401
