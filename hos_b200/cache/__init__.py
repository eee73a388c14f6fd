from .manager import CacheManager  # noqa: F401
from .pool import IdPool  # noqa: F401
