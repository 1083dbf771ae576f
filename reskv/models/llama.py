"""Alias: replaced by ``reskv_b200.models.hf_llama`` (``ResKVAttention``, ``ResKVForCausalLM``) on import."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("reskv_b200.models.hf_llama")
