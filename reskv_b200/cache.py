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
    """Cache of one attention layer (reference cache.py:10-103).

    Dense segment = ``sink_tokens`` attention sinks (the first tokens of the sequence, never compressed)
    followed by the sliding window; both live in one buffer ``[B, H, sinks + recent + group, 128]`` so that
    ``update`` can hand them to ``attention(..., recent=)`` as one tensor.  The compressed segment then
    starts at position ``sink_tokens``: pass ``start_position=layer.start_position`` to ``attention``.
    The reference's CUDA cache has no sinks (``sink_tokens=0``, the default, reproduces it); with sinks the
    split follows its accuracy path (reskv/accuracy.py:160-168): ``floor((T - recent - sinks) / group) *
    group`` prompt tokens are compressed, starting behind the sinks.
    """

    is_sliding = False

    def __init__(self, config: ResKVKernelConfig, sink_tokens: int = 0):
        super().__init__()
        if type(sink_tokens) is not int or sink_tokens < 0:
            raise ValueError("sink_tokens must be a non-negative integer")
        self.config = config
        self.sink_tokens = sink_tokens
        self.compressed = None
        self.raw_keys = None
        self.length = 0  # tokens seen
        self.live = 0    # tokens in the dense segment (sinks included)
        self.plan = None
        self._lib = None

    @property
    def start_position(self) -> int:
        """Position of the first compressed token (= number of sink tokens actually held)."""
        return min(self.sink_tokens, self.length)

    def lazy_initialization(self, key_states, value_states=None):
        from ._extension import bound_library

        b, h, _, d = key_states.shape
        slots = self.sink_tokens + self.config.recent_size + self.config.group_size
        # one allocation for the three window buffers
        window = torch.empty((3, b, h, slots, d), device=key_states.device, dtype=key_states.dtype)
        self.keys, self.raw_keys, self.values = window[0], window[1], window[2]
        self.plan = self.config.resolve(b)
        self._lib = bound_library(key_states.device)
        self.is_initialized = True

    def update(self, key_states, value_states, cache_kwargs=None, *args, **kwargs):
        """Append rotated keys / values (``cache_kwargs['raw_keys']`` = keys before
        RoPE).  Returns the dense segment ``(keys, values)``: sinks, then the window."""
        raw = (cache_kwargs or {}).get("raw_keys")
        if raw is None:
            raise ValueError("ResKV cache update requires pre-RoPE raw_keys")
        q_len = key_states.shape[2]
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        if self.length == 0:
            self._take_prompt(key_states, raw, value_states)
        elif q_len != 1:
            raise ValueError("ResKV continuation supports one token per step; chunked prefill is unsupported")
        else:
            self._take_token(key_states, raw, value_states)
        self.length += q_len
        return self.keys[:, :, : self.live], self.values[:, :, : self.live]

    def _take_prompt(self, keys, raw, values):
        """Split a prompt of T tokens into sinks [0, s), a compressed run [s, s + n) and the dense tail."""
        cfg, t = self.config, keys.shape[2]
        s = min(self.sink_tokens, t)
        n = max(0, t - cfg.recent_size - s) // cfg.group_size * cfg.group_size
        if n:
            # token slices of dense tensors go to the kernels as they are (token stride), no copy
            self.compressed = compress(raw[:, :, s : s + n], values[:, :, s : s + n], cfg, plan=self.plan)
        self.live = t - n
        if self.live > self.keys.shape[2]:
            raise ValueError("prefill leaves more dense tokens than the window holds")
        for buf, src in ((self.keys, keys), (self.raw_keys, raw), (self.values, values)):
            buf[:, :, :s].copy_(src[:, :, :s])
            buf[:, :, s : self.live].copy_(src[:, :, s + n :])

    def _take_token(self, key, raw, value):
        """One launch writes the token's rotated key, raw key and value into slot ``live`` of the three
        buffers; a full window then gives its oldest group to the compressed segment."""
        from ._extension import _stream, check

        b, h, cap, _ = self.keys.shape
        if key.dtype == torch.float16 and key.is_cuda:
            check(self._lib.reskv_window_write(self.keys.data_ptr(), self.raw_keys.data_ptr(), self.values.data_ptr(),
                                               key.contiguous().data_ptr(), raw.contiguous().data_ptr(),
                                               value.contiguous().data_ptr(), b, h, cap, self.live, _stream(key.device)))
        else:  # other dtypes (a BF16 model before its cast): plain slice copies
            at = self.live
            for buf, src in ((self.keys, key), (self.raw_keys, raw), (self.values, value)):
                buf[:, :, at : at + 1].copy_(src)
        self.live += 1
        if self.live == cap:
            self._compress_oldest_group()

    def _compress_oldest_group(self):
        s, n = self.sink_tokens, self.config.group_size
        self.compressed = compress(self.raw_keys[:, :, s : s + n], self.values[:, :, s : s + n], self.config,
                                   previous=self.compressed, plan=self.plan)
        remain = self.live - s - n
        if self.keys.dtype == torch.float16 and self.keys.is_cuda:
            from ._extension import _stream, check

            b, h, cap, _ = self.keys.shape
            check(self._lib.reskv_window_shift(self.keys.data_ptr(), self.raw_keys.data_ptr(), self.values.data_ptr(),
                                               b, h, cap, s, s + n, remain, _stream(self.keys.device)))
        else:
            for buf in (self.keys, self.raw_keys, self.values):
                tail = buf[:, :, s + n : self.live]
                buf[:, :, s : s + remain].copy_(tail if remain <= n else tail.clone())  # clone only when the ranges overlap
        self.live = s + remain

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

    def __init__(self, config: ResKVKernelConfig, num_layers: int, sink_tokens: int = 0):
        super().__init__(layers=[ResKVLayerCache(config, sink_tokens) for _ in range(num_layers)])

    def crop(self, max_length):
        raise NotImplementedError("ResKV does not support speculative cache rollback")

    def batch_repeat_interleave(self, repeats):
        for layer in self.layers:
            if layer.is_initialized:
                index = torch.arange(layer.keys.shape[0], device=layer.keys.device).repeat_interleave(repeats)
                layer.reorder_cache(index)

    def batch_select_indices(self, indices):
        self.reorder_cache(indices)
