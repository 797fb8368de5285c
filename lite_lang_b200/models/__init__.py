"""Architectures.  Importing this package registers each of them."""
from . import qwen2  # noqa: F401
from .qwen2 import Qwen2Config

__all__ = ["Qwen2Config"]
