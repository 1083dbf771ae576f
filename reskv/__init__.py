"""``reskv`` -- the reference package's name, served by ``reskv_b200``.

Code written against the reference (``from reskv import compress, attention``,
``from reskv.compression import cluster``, ``reskv._extension.load_extension`` ...)
imports this package unchanged and runs on the sm_100a library.  Every
sub-module here *is* the ``reskv_b200`` module of the same role (the entry in
``sys.modules`` is replaced, so ``reskv.config.KernelPlan is
reskv_b200.config.KernelPlan``).  Like the reference's ``__init__``
(reskv/__init__.py:18-39) nothing heavy is imported until a name is used:
the settings classes work without torch.
"""

from reskv_b200 import KernelPlan, ResKVConfig, ResKVKernelConfig, __version__  # noqa: F401

__all__ = ["ResKVKernelConfig", "ResKVForCausalLM", "ResKVConfig", "KernelPlan", "compress", "attention"]


class _AccuracySimulationModel:
    """Stands where the reference exports its accuracy-simulation models (reskv/models/accuracy.py): they
    evaluate compression error with dense tensors and are not part of the kernel hot path served here."""

    def __init__(self, *args, **kwargs):
        raise RuntimeError(f"{type(self).__name__}: the accuracy-simulation models are not part of this library; "
                           "it implements the compressed-KV kernel path (ResKVForCausalLM, compress, attention)")


def __getattr__(name):
    if name in ("ResKVLlamaAccuracyForCausalLM", "ResKVQwen3AccuracyForCausalLM"):
        return type(name, (_AccuracySimulationModel,), {})
    import reskv_b200

    try:
        return getattr(reskv_b200, name)
    except AttributeError:
        raise AttributeError(f"module 'reskv' has no attribute {name!r}") from None
