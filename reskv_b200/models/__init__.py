"""Model integration of the compressed KV cache.

``ResKVLlama`` is a self-contained Llama-shaped decoder (plain tensors, tensor parallel, CUDA-graph
decode); ``ResKVForCausalLM`` wraps Hugging Face Llama checkpoints (imported lazily: it needs
``transformers``).
"""

from .llama import LlamaShape, ResKVLlama

__all__ = ["LlamaShape", "ResKVLlama", "ResKVForCausalLM"]


def __getattr__(name):
    if name == "ResKVForCausalLM":
        from .hf_llama import ResKVForCausalLM

        return ResKVForCausalLM
    raise AttributeError(name)
