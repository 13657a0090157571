"""Architectures known to the registry."""
from . import qwen2  # noqa: F401
