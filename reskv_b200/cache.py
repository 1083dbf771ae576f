"""Two-segment KV cache of one layer: dense recent window + compressed segment.

Same behaviour as the reference cache (reskv/cache.py:10-122):

* prefill: the first ``floor((T - recent) / group) * group`` tokens are
  compressed (from position 0), the rest stays dense;
* decode: every token is appended to the dense window; when the window holds
  ``recent + group`` tokens its oldest ``group`` tokens are compressed with the
  existing centroid tables (``compress(..., previous=)``) and the window slides.

The window keeps rotated keys (for attention), raw pre-RoPE keys (for
compression) and values.  The compressed segment grows inside capacity buffers
(``CompressedTensor.append``), so a decode-time compression writes 64 tokens
instead of re-concatenating the whole segment.

The classes subclass the Hugging Face cache interfaces when ``transformers`` is
importable (method names follow transformers 5.x: ``lazy_initialization(key,
value)``, ``get_mask_sizes(query_length)``); without it they are plain objects
with the same methods.
"""

from __future__ import annotations

import torch

from .compression import compress
from .config import ResKVKernelConfig

try:  # optional: only needed to plug into Hugging Face models
    from transformers.cache_utils import Cache as _HFCache
    from transformers.cache_utils import CacheLayerMixin as _HFLayer
except Exception:  # pragma: no cover - transformers absent or incompatible
    _HFCache = _HFLayer = None


class _LayerBase:
    def __init__(self):
        self.keys = None
        self.values = None
        self.is_initialized = False


class ResKVLayerCache(_HFLayer or _LayerBase):
    """Cache of one attention layer (reference cache.py:10-103)."""

    is_sliding = False

    def __init__(self, config: ResKVKernelConfig):
        super().__init__()
        self.config = config
        self.compressed = None
        self.raw_keys = None
        self.length = 0  # tokens seen
        self.live = 0    # tokens in the dense window
        self.plan = None

    def lazy_initialization(self, key_states, value_states=None):
        b, h, _, d = key_states.shape
        slots = self.config.recent_size + self.config.group_size
        self.keys = torch.empty((b, h, slots, d), device=key_states.device, dtype=key_states.dtype)
        self.raw_keys = torch.empty_like(self.keys)
        self.values = torch.empty_like(self.keys)
        self.plan = self.config.resolve(b)
        self.is_initialized = True

    def update(self, key_states, value_states, cache_kwargs=None, *args, **kwargs):
        """Append rotated keys / values (``cache_kwargs['raw_keys']`` = keys before
        RoPE).  Returns the dense window ``(keys, values)``."""
        raw = (cache_kwargs or {}).get("raw_keys")
        if raw is None:
            raise ValueError("ResKV cache update requires pre-RoPE raw_keys")
        q_len = key_states.shape[2]
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        cfg = self.config
        if self.length == 0:
            n = max(0, q_len - cfg.recent_size) // cfg.group_size * cfg.group_size
            if n:
                self.compressed = compress(raw[:, :, :n].contiguous(), value_states[:, :, :n].contiguous(), cfg,
                                           plan=self.plan)
            self.live = q_len - n
            if self.live > self.keys.shape[2]:
                raise ValueError("prefill leaves more dense tokens than the window holds")
            self.keys[:, :, : self.live].copy_(key_states[:, :, n:])
            self.raw_keys[:, :, : self.live].copy_(raw[:, :, n:])
            self.values[:, :, : self.live].copy_(value_states[:, :, n:])
        else:
            if q_len != 1:
                raise ValueError("ResKV continuation supports one token per step; chunked prefill is unsupported")
            at = self.live
            self.keys[:, :, at : at + 1].copy_(key_states)
            self.raw_keys[:, :, at : at + 1].copy_(raw)
            self.values[:, :, at : at + 1].copy_(value_states)
            self.live += 1
            if self.live == self.keys.shape[2]:
                self._compress_oldest_group()
        self.length += q_len
        return self.keys[:, :, : self.live], self.values[:, :, : self.live]

    def _compress_oldest_group(self):
        n = self.config.group_size
        self.compressed = compress(self.raw_keys[:, :, :n].contiguous(), self.values[:, :, :n].contiguous(),
                                   self.config, previous=self.compressed, plan=self.plan)
        remain = self.live - n
        for buf in (self.keys, self.raw_keys, self.values):
            if remain <= n:
                buf[:, :, :remain].copy_(buf[:, :, n : self.live])  # source and target do not overlap
            else:
                buf[:, :, :remain].copy_(buf[:, :, n : self.live].clone())
        self.live = remain

    # -- Hugging Face cache-layer interface ---------------------------------------
    def get_seq_length(self):
        return self.length

    def get_mask_sizes(self, query_length):
        n = query_length if isinstance(query_length, int) else query_length.shape[0]
        return self.length + n, 0

    def get_max_cache_shape(self):
        return -1

    def reset(self):
        self.compressed = None
        self.length = self.live = 0
        self.keys = self.values = self.raw_keys = None
        self.plan = None
        self.is_initialized = False

    def reorder_cache(self, beam_idx):
        if self.is_initialized:
            index = beam_idx.to(self.keys.device)
            self.keys = self.keys.index_select(0, index)
            self.raw_keys = self.raw_keys.index_select(0, index)
            self.values = self.values.index_select(0, index)
            if self.compressed is not None:
                self.compressed.key = self.compressed.key.index_select(index)
                self.compressed.value = self.compressed.value.index_select(index)


class _CacheBase:
    def __init__(self, layers):
        self.layers = layers

    def reorder_cache(self, beam_idx):
        for layer in self.layers:
            layer.reorder_cache(beam_idx)


class ResKVCache(_HFCache or _CacheBase):
    """One ``ResKVLayerCache`` per layer (reference cache.py:106-122)."""

    def __init__(self, config: ResKVKernelConfig, num_layers: int):
        super().__init__(layers=[ResKVLayerCache(config) for _ in range(num_layers)])

    def crop(self, max_length):
        raise NotImplementedError("ResKV does not support speculative cache rollback")

    def batch_repeat_interleave(self, repeats):
        for layer in self.layers:
            if layer.is_initialized:
                index = torch.arange(layer.keys.shape[0], device=layer.keys.device).repeat_interleave(repeats)
                layer.reorder_cache(index)

    def batch_select_indices(self, indices):
        self.reorder_cache(indices)
