"""Settings objects for the compressed-KV hot path.

Three frozen dataclasses mirror the reference interface (reskv/config.py:8-248):

* ``ResKVKernelConfig`` -- what the user asks for (sparsity, bit width, mask
  layout, centroid fusion, clustering and cache sizes).
* ``KernelPlan`` -- what ``ResKVKernelConfig.resolve(batch)`` turns that into
  for one batch size; it travels with every ``CompressedTensor``.
* ``ResKVConfig`` -- the settings object of the reference's accuracy-simulation
  path.  Only the object is kept (``compress`` must reject it with a TypeError,
  and model checkpoints store it); the simulation itself is not part of this
  package.

Importing this module must not import torch (reference
tests/test_config.py:134-145), so it depends on the standard library only.

The ``tokens_per_warp`` / ``splits`` fields of a plan keep the reference's
values so that plans compare equal across the two implementations; the sm_100a
kernels treat ``splits`` as an upper-level hint (0 = choose from the SM count)
and ignore ``tokens_per_warp``, because their tiling is fixed at build time.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, fields

_LAYOUTS = ("unstructured", "tiled", "structured", "compact")
# "compact" has no counterpart in the reference: quantised residuals stored as bitmap + packed codes
# of the retained coordinates only (the reference's unstructured quantised layout stores all 128).
_FUSIONS = ("per_token", "deferred")


def _is_int(value) -> bool:
    # bool is an int subclass; the reference rejects it (config.py:38,94).
    return type(value) is int


@dataclass(frozen=True)
class ResKVConfig:
    """Settings of the accuracy-simulation path (reference config.py:8-54)."""

    sparsity: float = 0.75
    bits: int = 16
    num_clusters: int = 32
    recent_size: int = 32
    group_size: int = 64
    sink_tokens: int = 4
    kmeans_iterations: int = 15
    layout: str = "unstructured"

    def __post_init__(self):
        if isinstance(self.sparsity, bool) or self.sparsity not in (0.0, 0.5, 0.75, 0.875):
            raise ValueError("accuracy sparsity must be 0, 0.5, 0.75, or 0.875")
        if not _is_int(self.bits) or self.bits not in (2, 4, 8, 16):
            raise ValueError("accuracy bits must be 2, 4, 8, or 16 (16 disables quantization)")
        for name, floor, word in (
            ("num_clusters", 1, "positive"),
            ("group_size", 1, "positive"),
            ("kmeans_iterations", 1, "positive"),
            ("recent_size", 0, "nonnegative"),
            ("sink_tokens", 0, "nonnegative"),
        ):
            value = getattr(self, name)
            if not _is_int(value) or value < floor:
                raise ValueError(f"{name} must be a {word} integer")
        if self.layout not in ("unstructured", "structured"):
            raise ValueError("accuracy layout must be unstructured or structured")
        if self.layout == "structured" and self.sparsity != 0.75:
            raise ValueError("4:16 accuracy sparsity requires sparsity=0.75")

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class KernelPlan:
    """Resolved storage layout and decode schedule for one batch size.

    Mirrors reference config.py:198-248.  ``layout`` and ``bits`` decide the
    bytes a token occupies, ``centroid_fusion`` decides which decode kernel
    family reads them, ``nnz`` is the number of retained residual coordinates
    of a 128-wide head vector.
    """

    layout: str
    centroid_fusion: str
    bits: int
    nnz: int
    tokens_per_warp: int
    splits: int
    fixed_shift: bool = False

    def __post_init__(self):
        for name in ("bits", "nnz", "tokens_per_warp", "splits"):
            if not _is_int(getattr(self, name)):
                raise ValueError(f"{name} must be an integer")
        if type(self.fixed_shift) is not bool:
            raise ValueError("fixed_shift must be a boolean")
        if self.layout not in _LAYOUTS or self.bits not in (2, 4, 16):
            raise ValueError("invalid resolved layout or bit width")
        if self.centroid_fusion not in _FUSIONS or self.nnz not in (32, 64):
            raise ValueError("invalid resolved centroid fusion or retained dimension count")
        if self.tokens_per_warp not in (2, 4, 8, 12, 16) or self.splits < 0:
            raise ValueError("invalid warp or split schedule")
        if self.layout == "structured":
            if self.nnz != 32 or self.bits == 2:
                raise ValueError("invalid indexed residual configuration")
        elif self.layout == "tiled":
            if (self.bits, self.nnz, self.centroid_fusion) != (16, 64, "per_token"):
                raise ValueError("invalid tiled residual configuration")
        elif self.layout == "compact":
            if self.bits == 16 or self.nnz * self.bits < 128 or self.centroid_fusion != "per_token":
                raise ValueError("invalid compact residual configuration")
        else:
            wanted = "deferred" if self.bits == 16 else "per_token"
            if self.centroid_fusion != wanted:
                raise ValueError("invalid residual bit width and centroid fusion")
        if self.fixed_shift and (self.layout, self.bits, self.centroid_fusion) != (
            "structured",
            4,
            "deferred",
        ):
            raise ValueError("fixed shift requires indexed INT4 deferred fusion")

    def to_dict(self) -> dict:
        return asdict(self)


# (tokens_per_warp, splits) of the reference's schedule table (config.py:155-169).
# Kept only so that plans are equal across implementations.
def _reference_schedule(layout: str, fusion: str, bits: int, batch: int) -> tuple[int, int]:
    if layout == "structured":
        if bits == 4 and fusion == "deferred":
            return (4, 10) if batch >= 32 else (8, 14) if batch >= 8 else (4, 20)
        if bits == 4 and fusion == "per_token" and batch >= 8:
            return 4, 16
        return 4, 20
    if bits != 16:
        if batch <= 2:
            return 16, 40
        if batch <= 4:
            return 8, 20
        return (12, 0) if batch == 8 else (16, 0)
    return (4, 0) if fusion == "per_token" else (2, 0)


@dataclass(frozen=True)
class ResKVKernelConfig:
    """Compression and fused-decode settings (reference config.py:57-178).

    ``sparsity`` is the discarded fraction of residual coordinates (0.5 or
    0.75); ``bits`` 16 keeps FP16 residuals, 4 / 2 quantise them with one FP16
    scale per token; ``group_size`` is the number of *tokens* compressed
    together while decoding, ``recent_size`` the dense sliding window.
    """

    sparsity: float = 0.5
    bits: int = 16
    layout: str = "auto"
    centroid_fusion: str = "auto"
    num_clusters: int = 32
    max_clusters: int = 64
    group_size: int = 64
    recent_size: int = 32
    kmeans_iterations: int = 10
    rope_mode: str = "model"
    softmax_mode: str = "online"

    def __post_init__(self):
        for name in ("num_clusters", "max_clusters", "group_size", "recent_size", "kmeans_iterations"):
            if not _is_int(getattr(self, name)):
                raise ValueError(f"{name} must be an integer")
        if self.sparsity not in (0.5, 0.75):
            raise ValueError("sparsity must be 0.5 or 0.75 (discarded fraction)")
        if not _is_int(self.bits) or self.bits not in (2, 4, 16):
            raise ValueError("bits must be 2, 4, or 16 (FP16 sparse-only)")
        if self.layout not in ("auto",) + _LAYOUTS:
            raise ValueError("unknown sparsity layout")
        if self.centroid_fusion not in ("auto",) + _FUSIONS:
            raise ValueError("centroid_fusion must be auto, per_token or deferred")
        if not 1 <= self.num_clusters <= self.max_clusters <= 64:
            raise ValueError("require 1 <= num_clusters <= max_clusters <= 64")
        if self.group_size <= 0 or self.recent_size < 0 or self.kmeans_iterations <= 0:
            raise ValueError("group_size/iterations must be positive; recent_size nonnegative")
        if self.rope_mode not in ("model", "theta"):
            raise ValueError("rope_mode must be 'model' or 'theta'")
        if self.softmax_mode not in ("online", "fixed_shift"):
            raise ValueError("softmax_mode must be 'online' or 'fixed_shift'")
        if self.softmax_mode == "fixed_shift" and (self.bits, self.sparsity) != (4, 0.75):
            raise ValueError("fixed_shift softmax requires sparse75 INT4")
        if self.layout == "structured" and (self.sparsity != 0.75 or self.bits == 2):
            raise ValueError("structured layout requires sparsity=0.75 and bits=4 or 16")
        if self.layout == "tiled" and (self.bits, self.sparsity) != (16, 0.5):
            raise ValueError("tiled masks support only FP16 residuals at sparsity 0.5")
        if self.layout == "compact" and (self.bits == 16 or (self.bits == 2 and self.sparsity != 0.5)):
            raise ValueError("compact layout stores INT4 residuals, or INT2 residuals at sparsity 0.5")

    @property
    def keep_ratio(self) -> float:
        return 1.0 - self.sparsity

    def to_dict(self) -> dict:
        return asdict(self)

    def resolve(self, batch_size: int) -> KernelPlan:
        """Pick layout, centroid fusion and schedule for ``batch_size``.

        Defaults follow reference config.py:127-153: ``auto`` layout is the
        4:16 ``structured`` mask at sparsity 0.75 with 16- or 4-bit residuals
        and the ``unstructured`` bitmap otherwise; ``auto`` fusion is
        ``per_token`` for tiled masks, for quantised unstructured residuals and
        for structured masks at batch <= 2, else ``deferred``.
        """
        if not _is_int(batch_size) or batch_size < 1:
            raise ValueError("batch_size must be a positive integer")
        layout = self.layout
        if layout == "auto":
            layout = "structured" if (self.sparsity == 0.75 and self.bits != 2) else "unstructured"
        fusion = self.centroid_fusion
        if fusion == "auto":
            per_token = (
                layout in ("tiled", "compact")
                or (layout == "unstructured" and self.bits != 16)
                or (layout == "structured" and batch_size <= 2)
            )
            fusion = "per_token" if per_token else "deferred"
        if layout == "tiled" and fusion != "per_token":
            raise ValueError("tiled masks require per_token centroid fusion")
        if layout == "compact" and fusion != "per_token":
            raise ValueError("compact quantized caches require per_token centroid fusion")
        if layout == "unstructured":
            if self.bits == 16 and fusion != "deferred":
                raise ValueError("unstructured FP16 requires deferred centroid fusion")
            if self.bits != 16 and fusion != "per_token":
                raise ValueError("unstructured quantized caches require per_token centroid fusion")
        fixed = self.softmax_mode == "fixed_shift"
        if fixed and (layout, fusion) != ("structured", "deferred"):
            raise ValueError("fixed_shift requires structured layout with deferred centroid fusion")
        tpw, splits = _reference_schedule(layout, fusion, self.bits, batch_size)
        return KernelPlan(layout, fusion, self.bits, int(128 * self.keep_ratio), tpw, splits, fixed)


def _model_settings(model_config, settings, config_type, key):
    """Resolve the settings object of a model and store it back as a dict.

    Explicit ``settings`` win; otherwise ``model_config.<key>`` (a dict written
    by an earlier ``save_pretrained``) is decoded.  Anything that is not a dict
    of known field names is refused rather than replaced with defaults
    (reference config.py:181-195).
    """
    if settings is not None and not isinstance(settings, config_type):
        raise TypeError(f"expected {config_type.__name__}, got {type(settings).__name__}")
    if settings is None:
        stored = getattr(model_config, key, None)
        if stored is None:
            stored = {}
        known = {f.name for f in fields(config_type)}
        if not isinstance(stored, dict) or not set(stored) <= known:
            raise ValueError(
                f"checkpoint compression settings do not match {config_type.__name__}; "
                "pass an explicit configuration"
            )
        settings = config_type(**stored)
    setattr(model_config, key, settings.to_dict())
    return settings
