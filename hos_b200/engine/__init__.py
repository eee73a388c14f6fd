from .engine import Engine  # noqa: F401
from .runner import Runner  # noqa: F401
