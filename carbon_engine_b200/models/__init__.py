"""Architectures the engine can build.  Importing this package registers them."""
from . import qwen3  # noqa: F401
