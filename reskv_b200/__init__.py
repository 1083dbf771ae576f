"""B200-native implementation of the ResKV compressed-KV hot path.

Same public names as the reference package (reskv/__init__.py:4-39):
``ResKVKernelConfig``, ``ResKVConfig``, ``compress``, ``attention``; the
settings classes import without torch, everything that touches CUDA is loaded
on first use.
"""

from .config import KernelPlan, ResKVConfig, ResKVKernelConfig

__version__ = "0.1.0"
__all__ = ["ResKVKernelConfig", "ResKVForCausalLM", "ResKVConfig", "KernelPlan", "compress", "attention"]


def __getattr__(name):
    if name == "compress":
        from .compression import compress

        return compress
    if name == "attention":
        from ._attention import attention

        return attention
    if name == "ResKVForCausalLM":  # needs transformers: imported on first use (reference __init__.py:18-21)
        from .models.hf_llama import ResKVForCausalLM

        return ResKVForCausalLM
    raise AttributeError(name)
