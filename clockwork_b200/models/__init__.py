"""Architectures.  Importing this package registers each of them by name."""

from . import qwen2  # noqa: F401
from .qwen2 import Qwen2Architecture, Qwen2Config

__all__ = ["Qwen2Architecture", "Qwen2Config"]
