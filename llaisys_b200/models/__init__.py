"""Model wrappers (reference: python/llaisys/models/__init__.py:1)."""
from .qwen2 import Qwen2

__all__ = ["Qwen2"]
