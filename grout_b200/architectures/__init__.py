"""Architectures known to the library; importing this package registers them."""
from . import qwen3  # noqa: F401
