"""Model integration of the compressed KV cache."""

from .llama import LlamaShape, ResKVLlama

__all__ = ["LlamaShape", "ResKVLlama"]
