"""Alias: this module is replaced by ``reskv_b200.compression`` on import."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("reskv_b200.compression")
