"""Storage format of one compressed K or V cache.

``CompressedTensor`` / ``CompressedKV`` keep the field names, shapes, dtypes and
error behaviour of the reference containers (reskv/tensors.py:11-162) so that
code written against them keeps working:

=================  ===========================================================
field              contents, for ``B`` sequences, ``H`` KV heads, ``T`` tokens
=================  ===========================================================
``centroids``      FP16 ``[B,H,C,128]``, ``1 <= C <= 64``
``cluster_ids``    integer ``[B,H,T]`` on entry, held as int8
``payload``        FP16 ``[B,H,T,nnz]`` (bits 16), or int32 words: 4 (structured
                   INT4) / ``4*bits`` (unstructured INT4/INT2, all 128 coords)
``metadata``       int64 ``[B,H,T,2]`` bitmap, MSB first (unstructured FP16);
                   int32 ``[B,H,T,4]`` (tiled / structured FP16);
                   int32 ``[B,H,T,2]`` (structured INT4); ``None`` otherwise
``scale``          FP16 ``[B,H,T]`` for quantised residuals, else ``None``
=================  ===========================================================

What differs from the reference is how the token axis is stored.  The reference
re-concatenates every tensor whenever a decode group is appended
(tensors.py:105-119).  Here the per-token tensors may be *windows* of larger
buffers whose token axis has spare capacity: ``append`` writes the new group
behind the live tokens and returns a longer window over the same memory,
doubling the buffers only when they are full.  The kernels therefore take a
token stride (tokens of capacity per ``(b, h)`` unit) next to the token count,
and ``_native`` holds ``[B*H, T, w]`` views that need not be contiguous across
units.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .config import KernelPlan

_INT_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64)


def payload_width(plan: KernelPlan) -> int:
    """Last-axis length of ``payload`` for ``plan`` (reference tensors.py:58-64)."""
    if plan.bits == 16:
        return plan.nnz
    if plan.layout == "compact":
        return plan.nnz * plan.bits // 32  # codes of the retained coordinates only
    return 4 if plan.layout == "structured" else 4 * plan.bits


def metadata_spec(plan: KernelPlan):
    """``(words, dtype)`` of ``metadata`` for ``plan``, or ``None`` when unused."""
    if plan.bits != 16 and plan.layout not in ("structured", "compact"):
        return None
    if plan.layout in ("unstructured", "compact"):
        return 2, torch.int64
    return (2 if plan.bits == 4 else 4), torch.int32


@dataclass
class CompressedTensor:
    """Compressed K or V cache of one layer; see the module docstring."""

    centroids: torch.Tensor
    cluster_ids: torch.Tensor
    payload: torch.Tensor
    metadata: torch.Tensor | None
    scale: torch.Tensor | None
    plan: KernelPlan
    _native: tuple = field(default=(), init=False, repr=False)
    # Backing buffers [B,H,capacity,...] of (ids, payload, metadata, scale); the
    # public fields are their leading ``T`` tokens.
    _buffers: tuple = field(default=(), init=False, repr=False)
    # One-element list shared by every window over the same ``_buffers``: the number of tokens that
    # some window has already written there.  A window shorter than that has a sibling that appended
    # first, so its own ``append`` must not write into the shared buffers (it copies instead).
    _live: list = field(default=None, init=False, repr=False)
    _flat: tuple = field(default=(), init=False, repr=False)  # ``_buffers`` as [B*H, capacity, ...] views

    def __post_init__(self):
        c, ids, p = self.centroids, self.cluster_ids, self.payload
        if c.ndim != 4 or c.shape[-1] != 128:
            raise ValueError("centroids must have shape [B,H,C,128]")
        if ids.ndim != 3 or ids.shape[:2] != c.shape[:2]:
            raise ValueError("cluster IDs must have shape [B,H,T]")
        if not 1 <= c.shape[2] <= 64:
            raise ValueError("centroid count must be between 1 and 64")
        if p.ndim != 4 or p.shape[:3] != ids.shape:
            raise ValueError("payload must have shape [B,H,T,words_or_values]")
        for t in (ids, p, self.metadata, self.scale):
            if t is not None and t.device != c.device:
                raise ValueError("all cache tensors must share a device")
        if c.dtype != torch.float16:
            raise ValueError("centroids must be FP16")
        plan = self.plan
        if p.dtype != (torch.float16 if plan.bits == 16 else torch.int32):
            raise ValueError("payload dtype does not match the compression plan")
        b, h, n = ids.shape
        if min(b, h, n) < 1:
            raise ValueError("cache dimensions must be nonempty")
        if ids.dtype not in _INT_DTYPES:
            raise ValueError("cluster IDs must be integer tensors")
        if p.shape[-1] != payload_width(plan):
            raise ValueError("payload width does not match the compression plan")
        spec = metadata_spec(plan)
        if spec is not None:
            words, dtype = spec
            m = self.metadata
            if m is None or m.shape != (b, h, n, words) or m.dtype != dtype:
                raise ValueError("sparse metadata shape/dtype does not match the compression plan")
        elif self.metadata is not None:
            raise ValueError("quantized unstructured payloads do not use sparse metadata")
        if plan.bits != 16:
            s = self.scale
            if s is None or s.shape != (b, h, n) or s.dtype != torch.float16:
                raise ValueError("quantized scales must be FP16 [B,H,T]")
        elif self.scale is not None:
            raise ValueError("FP16 sparse-only caches do not use quantization scales")
        if not self._buffers:
            # Plain tensors: they are their own buffers, capacity == T.
            self.cluster_ids = ids.to(torch.int8).contiguous()
            self.payload = p.contiguous()
            self.metadata = self.metadata.contiguous() if self.metadata is not None else None
            self.scale = self.scale.contiguous() if self.scale is not None else None
            self._buffers = (self.cluster_ids, self.payload, self.metadata, self.scale)
            self._live = [n]
        self._native = self._native_views(c, n)

    def _native_views(self, centroids, n: int) -> tuple:
        """What the kernels are given: the centroid table as ``[B*H, C, 128]`` and the first ``n`` tokens of every
        capacity buffer as ``[B*H, n, w]`` (``[B*H, n]`` for ids and scales)."""
        b, h, cap = self._buffers[0].shape[:3]
        if not self._flat:  # the buffers with (B, H) merged: made once per set of buffers, windows share them
            self._flat = tuple(None if buf is None else buf.reshape(b * h, cap, -1).squeeze(-1) if buf.ndim == 3
                               else buf.reshape(b * h, cap, -1) for buf in self._buffers)
        return (centroids.reshape(b * h, -1, 128).contiguous(),
                *(None if flat is None else flat.narrow(1, 0, n) for flat in self._flat))

    def _grown(self, centroids, length: int) -> "CompressedTensor":
        """Window over the first ``length`` tokens of this tensor's own buffers with a newer centroid table, for
        library calls that have just written tokens ``[seq_len, length)`` there: same plan, same buffers, same
        written-length marker, nothing to validate again."""
        new = CompressedTensor.__new__(CompressedTensor)
        new.centroids, new.plan, new._buffers, new._live = centroids, self.plan, self._buffers, self._live
        new._flat = self._flat
        new.cluster_ids, new.payload, new.metadata, new.scale = (
            None if buf is None else buf.narrow(2, 0, length) for buf in self._buffers)
        new._native = new._native_views(centroids, length)
        return new

    @classmethod
    def _window(cls, centroids, buffers, length, plan, live=None) -> "CompressedTensor":
        """Tensor over the first ``length`` tokens of capacity ``buffers``; ``live`` is the written-length
        marker of those buffers (a fresh one when they are new)."""
        self = cls.__new__(cls)
        self.centroids = centroids
        self.plan = plan
        self._buffers = tuple(buffers)
        self._flat = ()
        self._live = [length] if live is None else live
        views = [buf[:, :, :length] if buf is not None else None for buf in buffers]
        self.cluster_ids, self.payload, self.metadata, self.scale = views
        self._native = ()
        self.__post_init__()
        return self

    # -- queries ----------------------------------------------------------
    @property
    def seq_len(self) -> int:
        return self.cluster_ids.shape[-1]

    @property
    def token_stride(self) -> int:
        """Tokens between consecutive ``(b, h)`` units in the backing buffers."""
        return self._buffers[0].shape[2]

    @property
    def tensors(self) -> tuple:
        """All stored tensors, including the flattened views passed to the kernels."""
        return (self.centroids, self.cluster_ids, self.payload, self.metadata, self.scale, *self._native)

    @property
    def nbytes(self) -> int:
        """Bytes of the backing storages, i.e. of the *capacity* (up to twice the live data after an
        ``append`` grew the buffers); ``live_nbytes`` counts the live tokens only."""
        return _storage_bytes(self.tensors)

    @property
    def live_nbytes(self) -> int:
        """Bytes the live tokens occupy (what the reference's ``nbytes`` reports for its exactly sized
        tensors, reskv/tensors.py:121-132): centroid table plus ``seq_len`` rows of every per-token tensor."""
        views = (self.centroids, self.cluster_ids, self.payload, self.metadata, self.scale)
        return sum(v.numel() * v.element_size() for v in views if v is not None)

    # -- updates ----------------------------------------------------------
    def reserve(self, capacity: int, *, copy: bool = False) -> "CompressedTensor":
        """Same tokens over buffers that hold at least ``capacity`` tokens (``copy=True``: over new
        buffers even when the present ones are large enough)."""
        n = self.seq_len
        if self.token_stride >= capacity and not copy:
            return self
        return _regrow([self], max(capacity, n))[0]

    def append(self, other: "CompressedTensor") -> "CompressedTensor":
        """Tokens of ``self`` followed by those of ``other``.

        The newer centroid table replaces the older one (reference
        tensors.py:105-119).  Where the reference concatenates, this writes
        ``other`` behind the live tokens of ``self``'s buffers and returns a
        longer window over the same memory; only a full buffer is reallocated
        (to twice the needed length).  ``self`` stays valid: its tokens are not
        touched.  Appending twice to the same tensor (two continuations of one
        prefix) is as functional as the reference's ``torch.cat``: the second
        append finds the slots behind ``self`` taken by the first and writes into
        a copy, so both results stay intact.
        """
        if self.plan != other.plan:
            raise ValueError("cannot concatenate different cache plans")
        n, total = self.seq_len, self.seq_len + other.seq_len
        taken = self._live[0] != n  # a sibling window already appended behind these tokens
        base = self
        if taken or self.token_stride < total:
            base = self.reserve(max(2 * total, 256) if self.token_stride < total else self.token_stride, copy=taken)
        news = (other.cluster_ids, other.payload, other.metadata, other.scale)
        for buf, new in zip(base._buffers, news):
            if buf is not None:
                buf[:, :, n:total].copy_(new)
        base._live[0] = total
        return CompressedTensor._window(other.centroids, base._buffers, total, self.plan, base._live)

    def index_select(self, index: torch.Tensor) -> "CompressedTensor":
        def take(t):
            return t.index_select(0, index.to(t.device)) if t is not None else None

        return CompressedTensor(
            take(self.centroids),
            take(self.cluster_ids),
            take(self.payload),
            take(self.metadata),
            take(self.scale),
            self.plan,
        )


@dataclass
class CompressedKV:
    """The compressed keys and values of one layer (reference tensors.py:135-152)."""

    key: CompressedTensor
    value: CompressedTensor

    def __post_init__(self):
        if self.key.plan != self.value.plan or self.key.cluster_ids.shape != self.value.cluster_ids.shape:
            raise ValueError("K/V compression plans and token dimensions must agree")
        if self.key.centroids.device != self.value.centroids.device:
            raise ValueError("K/V caches must share a device")

    @property
    def seq_len(self) -> int:
        return self.key.seq_len

    @property
    def nbytes(self) -> int:
        return _storage_bytes((*self.key.tensors, *self.value.tensors))

    def reserve(self, capacity: int) -> "CompressedKV":
        """Both sides over buffers of at least ``capacity`` tokens, grown together in one allocation."""
        if min(self.key.token_stride, self.value.token_stride) >= capacity:
            return self
        return CompressedKV(*_regrow([self.key, self.value], max(capacity, self.seq_len)))


def _regrow(tensors, capacity: int):
    """The given compressed tensors over fresh buffers of ``capacity`` tokens, all carved from ONE allocation (every
    buffer starts on a 256-byte boundary): a layer's cache then costs one trip to the device allocator."""
    plans = []
    for ct in tensors:
        b, h = ct.cluster_ids.shape[:2]
        for view in (ct.cluster_ids, ct.payload, ct.metadata, ct.scale):
            used = 0 if view is None else b * h * capacity * view[0, 0, 0].numel() * view.element_size()
            plans.append((view, used, -(-used // 256) * 256))
    arena = torch.empty(sum(size for _, _, size in plans), dtype=torch.uint8, device=tensors[0].cluster_ids.device)
    out, at, it = [], 0, iter(plans)
    for ct in tensors:
        b, h = ct.cluster_ids.shape[:2]
        n, grown = ct.seq_len, []
        for _ in range(4):
            view, used, size = next(it)
            if view is None:
                grown.append(None)
                continue
            buf = arena[at : at + used].view(view.dtype).view((b, h, capacity) + tuple(view.shape[3:]))
            buf[:, :, :n].copy_(view)
            grown.append(buf)
            at += size
        out.append(CompressedTensor._window(ct.centroids, grown, n, ct.plan))
    return out


def _storage_bytes(tensors) -> int:
    """Bytes in distinct backing storages; views of one storage count once."""
    seen = {}
    for t in tensors:
        if isinstance(t, torch.Tensor):
            s = t.untyped_storage()
            seen[(t.device, s.data_ptr())] = s.nbytes()
    return sum(seen.values())
