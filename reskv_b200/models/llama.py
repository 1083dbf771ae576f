"""Llama-architecture decoder that keeps its KV cache compressed.

Counterpart of the reference's ``ResKVForCausalLM`` (reskv/models/llama.py:25-170):
prefill attends to dense K/V (SDPA) and then compresses them, decode steps call
the fused compressed attention with the dense recent window.  The reference
subclasses the Hugging Face model; this one is a self-contained module over
plain weight tensors so that it does not depend on a transformers version, can
run with random weights of any Llama shape (the benchmarks need no checkpoint)
and can be tensor-parallel: query/KV heads and the FFN are split over the ranks
(every rank keeps the caches of its own KV heads, so compression and attention
stay local) and the only collectives are the sum all-reduces after ``o_proj``
and ``down_proj``.

``cache="dense"`` keeps an ordinary FP16 KV cache instead (SDPA decode): the
baseline the compressed path is measured against.

Dense matrix products use torch (cuBLAS); everything that touches the
compressed cache goes through ``reskv_b200.compress`` / ``attention``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .._attention import attention
from ..cache import ResKVLayerCache
from ..config import ResKVKernelConfig

try:  # dense baseline only: library flash-decoding kernel, if the image has it
    from flash_attn import flash_attn_with_kvcache as _flash_kvcache
except Exception:  # pragma: no cover
    _flash_kvcache = None


@dataclass(frozen=True)
class LlamaShape:
    """Architecture sizes; defaults are Llama-3.1-8B."""

    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5


def _rms_norm(x, weight, eps):
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return (v * weight.float()).to(x.dtype)


def _rope(x, cos, sin):
    """Half-split RoPE; x [B, H, T, 128], cos/sin [T, 64] (FP32)."""
    a, b = x.float()[..., :64], x.float()[..., 64:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1).to(x.dtype)


class _DenseLayerCache:
    """Plain FP16 KV cache of one layer (rotated keys), preallocated."""

    def __init__(self, batch, kv_heads, capacity, device):
        self.k = torch.empty((batch, kv_heads, capacity, 128), dtype=torch.float16, device=device)
        self.v = torch.empty_like(self.k)
        self.length = 0

    def append(self, k_rot, v):
        n = k_rot.shape[2]
        self.k[:, :, self.length:self.length + n].copy_(k_rot)
        self.v[:, :, self.length:self.length + n].copy_(v)
        self.length += n
        return self.k[:, :, :self.length], self.v[:, :, :self.length]


class ResKVLlama:
    """Random-weight or loaded Llama decoder with a compressed (or dense) KV cache.

    ``generate(ids, new_tokens)`` = prefill + greedy decode.  With a process
    group the model is tensor-parallel over ``group`` (heads and FFN columns are
    sharded; ``shape.kv_heads`` must be divisible by the group size).
    """

    def __init__(self, shape: LlamaShape = LlamaShape(), kernel_config: ResKVKernelConfig | None = None, *,
                 cache: str = "reskv", device="cuda", seed: int = 0, group=None, prefill_chunk: int = 65536,
                 sink_tokens: int = 0):
        if cache not in ("reskv", "dense"):
            raise ValueError("cache must be 'reskv' or 'dense'")
        self.shape, self.cache_kind, self.device = shape, cache, torch.device(device)
        self.kernel_config = kernel_config or ResKVKernelConfig()
        if not isinstance(self.kernel_config, ResKVKernelConfig):
            raise TypeError(f"expected ResKVKernelConfig, got {type(self.kernel_config).__name__}")
        self.sink_tokens = int(sink_tokens)  # leading tokens kept dense (attention sinks); compression starts behind them
        self.group = group
        self.tp = 1 if group is None else torch.distributed.get_world_size(group)
        if shape.kv_heads % self.tp or shape.heads % self.tp or shape.ffn % self.tp:
            raise ValueError("heads, kv_heads and ffn must be divisible by the tensor-parallel size")
        self.h_q, self.h_kv, self.ffn = shape.heads // self.tp, shape.kv_heads // self.tp, shape.ffn // self.tp
        self.prefill_chunk = prefill_chunk
        rank = 0 if group is None else torch.distributed.get_rank(group)
        g = torch.Generator(device=self.device).manual_seed(seed)

        def w(rows, cols, std):
            # every rank draws the full matrix from the same seed and keeps its shard, so the
            # model is the same function for every tensor-parallel size
            return (torch.randn(rows, cols, generator=g, device=self.device, dtype=torch.float32) * std).half()

        def rows_of(full, per_rank):
            return full[rank * per_rank:(rank + 1) * per_rank].contiguous()

        d, hd = shape.hidden, shape.head_dim
        self.embed = w(shape.vocab, d, 1.0)
        self.lm_head = w(shape.vocab, d, d**-0.5)
        self.final_norm = torch.ones(d, dtype=torch.float16, device=self.device)
        self.layers = []
        for _ in range(shape.layers):
            wq, wk, wv = w(shape.heads * hd, d, d**-0.5), w(shape.kv_heads * hd, d, d**-0.5), w(shape.kv_heads * hd, d, d**-0.5)
            wo = w(d, shape.heads * hd, (shape.heads * hd) ** -0.5)
            wg, wu = w(shape.ffn, d, d**-0.5), w(shape.ffn, d, d**-0.5)
            wd = w(d, shape.ffn, shape.ffn**-0.5)
            self.layers.append({
                "norm1": torch.ones(d, dtype=torch.float16, device=self.device),
                "norm2": torch.ones(d, dtype=torch.float16, device=self.device),
                # [q | k | v] rows of this rank's heads ([out, in] for F.linear)
                "wqkv": torch.cat((rows_of(wq, self.h_q * hd), rows_of(wk, self.h_kv * hd), rows_of(wv, self.h_kv * hd))),
                "wo": wo[:, rank * self.h_q * hd:(rank + 1) * self.h_q * hd].contiguous(),
                "w_gate_up": torch.cat((rows_of(wg, self.ffn), rows_of(wu, self.ffn))),
                "w_down": wd[:, rank * self.ffn:(rank + 1) * self.ffn].contiguous(),
            })
            del wq, wk, wv, wo, wg, wu, wd
        self.inv_freq = (shape.rope_theta ** (-torch.arange(64, device=self.device).float() / 64)).contiguous()
        self.scaling = hd**-0.5
        self.caches = None
        self.length = 0

    # -- helpers -----------------------------------------------------------------------------
    def _all_reduce(self, x):
        if self.tp > 1:
            torch.distributed.all_reduce(x, group=self.group)
        return x

    def _trig(self, start, n):
        ang = torch.arange(start, start + n, device=self.device).float()[:, None] * self.inv_freq[None, :]
        return ang.cos(), ang.sin()

    def _mlp(self, layer, x):
        out = torch.empty_like(x)
        flat, oflat = x.reshape(-1, x.shape[-1]), out.reshape(-1, x.shape[-1])
        for i in range(0, flat.shape[0], self.prefill_chunk):
            gu = F.linear(flat[i:i + self.prefill_chunk], layer["w_gate_up"])
            gate = F.silu(gu[:, :self.ffn])
            gate.mul_(gu[:, self.ffn:])
            oflat[i:i + self.prefill_chunk] = F.linear(gate, layer["w_down"])
        return self._all_reduce(out)

    def _qkv(self, layer, x):
        b, t, _ = x.shape
        qkv = F.linear(_rms_norm(x, layer["norm1"], self.shape.rms_eps), layer["wqkv"])
        q, k, v = qkv.split((self.h_q * 128, self.h_kv * 128, self.h_kv * 128), dim=-1)
        return (q.reshape(b, t, self.h_q, 128).transpose(1, 2), k.reshape(b, t, self.h_kv, 128).transpose(1, 2),
                v.reshape(b, t, self.h_kv, 128).transpose(1, 2).contiguous())

    # -- prefill / decode ----------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, reserve: int = 0) -> torch.Tensor:
        """Run the prompt ``ids [B, T]``; builds the caches; returns last-token logits.

        Norms, projections, RoPE and the dense causal attention run over slices of the batch (at most
        ``prefill_chunk`` tokens at a time) so that their FP32 temporaries stay small at long contexts;
        the cache of a layer receives the whole batch at once."""
        b, t = ids.shape
        cos, sin = self._trig(0, t)
        x = self.embed[ids]
        self.caches = []
        rows = max(1, self.prefill_chunk // t)  # sequences per slice
        half = dict(dtype=torch.float16, device=self.device)
        for layer in self.layers:
            k_raw = torch.empty((b, self.h_kv, t, 128), **half)
            k_rot, v_all = torch.empty_like(k_raw), torch.empty_like(k_raw)
            att = torch.empty((b, t, self.h_q * 128), **half)
            for i in range(0, b, rows):
                q, k, v = self._qkv(layer, x[i:i + rows])
                qr, kr = _rope(q, cos, sin), _rope(k, cos, sin)
                out = F.scaled_dot_product_attention(qr, kr, v, is_causal=t > 1, enable_gqa=True, scale=self.scaling)
                att[i:i + rows] = out.transpose(1, 2).reshape(-1, t, self.h_q * 128)
                k_raw[i:i + rows], k_rot[i:i + rows], v_all[i:i + rows] = k, kr, v
                del q, k, v, qr, kr, out
            if self.cache_kind == "reskv":
                cache = ResKVLayerCache(self.kernel_config, self.sink_tokens)
                cache.update(k_rot, v_all, {"raw_keys": k_raw})
                if reserve and cache.compressed is not None:
                    cache.compressed = cache.compressed.reserve(cache.compressed.seq_len + reserve)
            else:
                cache = _DenseLayerCache(b, self.h_kv, t + reserve, self.device)
                cache.append(k_rot, v_all)
            self.caches.append(cache)
            del k_raw, k_rot, v_all
            for i in range(0, b, rows):
                x[i:i + rows] += self._all_reduce(F.linear(att[i:i + rows], layer["wo"]))
            del att
            for i in range(0, b, rows):
                x[i:i + rows] += self._mlp(layer, _rms_norm(x[i:i + rows], layer["norm2"], self.shape.rms_eps))
        self.length = t
        return self._logits(x[:, -1:])

    def _logits(self, x):
        return F.linear(_rms_norm(x, self.final_norm, self.shape.rms_eps), self.lm_head)[:, 0].float()

    @torch.no_grad()
    def decode(self, tokens: torch.Tensor) -> torch.Tensor:
        """One step for ``tokens [B]``; returns logits ``[B, vocab]``."""
        b = tokens.shape[0]
        pos = self.length
        cos, sin = self._trig(pos, 1)
        x = self.embed[tokens].unsqueeze(1)
        for layer, cache in zip(self.layers, self.caches):
            q, k, v = self._qkv(layer, x)
            qr, kr = _rope(q, cos, sin), _rope(k, cos, sin)
            if self.cache_kind == "reskv":
                keys, values = cache.update(kr, v, {"raw_keys": k.contiguous()})
                if cache.compressed is not None:
                    att = attention(q.contiguous(), cache.compressed, position=pos, start_position=cache.start_position,
                                    inv_freq=self.inv_freq, scaling=self.scaling, recent=(qr, keys, values))
                else:
                    att = F.scaled_dot_product_attention(qr, keys, values, enable_gqa=True, scale=self.scaling)
            else:
                keys, values = cache.append(kr, v)
                att = F.scaled_dot_product_attention(qr, keys, values, enable_gqa=True, scale=self.scaling)
            x = x + self._all_reduce(F.linear(att.transpose(1, 2).reshape(b, 1, -1), layer["wo"]))
            x = x + self._mlp(layer, _rms_norm(x, layer["norm2"], self.shape.rms_eps))
        self.length += 1
        return self._logits(x)

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy continuation ``[B, new_tokens]`` of the prompt ``ids [B, T]``."""
        logits = self.prefill(ids, reserve=new_tokens)
        out = [logits.argmax(-1)]
        for _ in range(new_tokens - 1):
            out.append(self.decode(out[-1]).argmax(-1))
        return torch.stack(out, dim=1)

    # -- CUDA-graph decode ------------------------------------------------------------------------
    # A decode step is ~20 small launches per layer; at small batch the GPU waits for Python.  The
    # step is therefore captured once per "epoch" (the 64 steps between two group compressions, in
    # which the compressed segment is fixed) and replayed: query position and window length live in
    # a device-side step state that the append / decode kernels read and a final kernel advances.
    def _step_body(self, tok):
        from .._extension import (LAYOUT_COMPACT, LAYOUT_STRUCTURED, LAYOUT_TILED, LAYOUT_UNSTRUCTURED, _stream,
                                  bound_library, check)

        lib = bound_library(self.device)  # every launch below runs with the model's device current
        b = tok.shape[0]
        d = self.shape.hidden
        stream = _stream(self.device)
        state = self._state.data_ptr()
        reskv = self.cache_kind == "reskv"

        def half(*shape):
            return torch.empty(shape, dtype=torch.float16, device=self.device)

        def norm(x, weight):
            out = half(b, d)
            check(lib.reskv_rms_norm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), b, d, float(self.shape.rms_eps), stream))
            return out

        def ptr(t):
            return None if t is None else t.data_ptr()

        def project(x, inp, weight):
            """x + inp @ weight^T, summed over the tensor-parallel group."""
            if self.tp == 1:
                return torch.addmm(x, inp, weight.t())
            return x + self._all_reduce(F.linear(inp, weight))

        if reskv:
            # count the new token into the window first: it goes to slot count - 1 and the
            # attention of this step already includes it
            check(lib.reskv_step_advance(state, 0, 1, stream))
        x = self.embed[tok]
        for index, (layer, cache) in enumerate(zip(self.layers, self.caches)):
            qkv = F.linear(norm(x, layer["norm1"]), layer["wqkv"])
            q_rot = half(b * self.h_q, 128)
            if reskv:
                cap = cache.keys.shape[2]
                q_raw = half(b * self.h_q, 128)
                check(lib.reskv_rope_split(qkv.data_ptr(), b, self.h_q, self.h_kv, self.inv_freq.data_ptr(), state,
                                           q_raw.data_ptr(), q_rot.data_ptr(), None, None, cache.keys.data_ptr(),
                                           cache.raw_keys.data_ptr(), cache.values.data_ptr(), cap, stream))
                key, val = cache.compressed.key, cache.compressed.value
                plan = key.plan
                _, ki, kp, km, ks = key._native
                _, vi, vp, vm, vs = val._native
                kc, vc = self._centroids[index]
                layout = {"unstructured": LAYOUT_UNSTRUCTURED, "tiled": LAYOUT_TILED, "structured": LAYOUT_STRUCTURED,
                          "compact": LAYOUT_COMPACT}[plan.layout]
                att = half(b, self.h_q * 128)
                # token count and centroid tables are read from the step state / fixed-shape tables,
                # so the captured launch stays valid when a group is compressed between replays
                check(lib.reskv_decode_step(layout, plan.bits, plan.nnz, q_raw.data_ptr(), kc.data_ptr(), ki.data_ptr(),
                                            kp.data_ptr(), ptr(km), ptr(ks), vc.data_ptr(), vi.data_ptr(), vp.data_ptr(),
                                            ptr(vm), ptr(vs), b, self.h_kv, self.h_q, key.seq_len, key.token_stride,
                                            kc.shape[1], vc.shape[1], cache.start_position, float(self.shape.rope_theta),
                                            self.inv_freq.data_ptr(), float(self.scaling), 0, q_rot.data_ptr(),
                                            cache.keys.data_ptr(), cache.values.data_ptr(), cap, state,
                                            self._workspace.data_ptr(), self._workspace.numel(), att.data_ptr(), stream),
                      launches=2)
            elif _flash_kvcache is not None:
                k_rot, v_new = half(b, 1, self.h_kv, 128), half(b, 1, self.h_kv, 128)
                check(lib.reskv_rope_split(qkv.data_ptr(), b, self.h_q, self.h_kv, self.inv_freq.data_ptr(), state,
                                           None, q_rot.data_ptr(), k_rot.data_ptr(), v_new.data_ptr(), None, None, None,
                                           0, stream))
                att = _flash_kvcache(q_rot.view(b, 1, self.h_q, 128), cache.k, cache.v, k=k_rot, v=v_new,
                                     cache_seqlens=self._seqlens, softmax_scale=self.scaling, causal=True)
                att = att.reshape(b, self.h_q * 128)
            else:
                raise RuntimeError("graph decode of the dense baseline needs flash_attn")
            x = project(x, att, layer["wo"])
            gate_up = F.linear(norm(x, layer["norm2"]), layer["w_gate_up"])
            act = half(b, self.ffn)
            check(lib.reskv_silu_mul(gate_up.data_ptr(), act.data_ptr(), b, self.ffn, stream))
            x = project(x, act, layer["w_down"])
        check(lib.reskv_step_advance(state, 1, 0, stream))
        if not reskv:
            self._seqlens += 1
        return F.linear(norm(x, self.final_norm), self.lm_head).float()

    @torch.no_grad()
    def begin_graph_decode(self, batch: int):
        """Prepare static buffers after ``prefill``; call once before ``decode_graph``."""
        from .._extension import library

        self._tok_in = torch.zeros(batch, dtype=torch.long, device=self.device)
        self._graph = None
        self._warmed = False
        if self.cache_kind == "reskv":
            self._state = torch.zeros(4, dtype=torch.int32, device=self.device)
            # centroid tables at their final shape (zero rows beyond the live count), one pair per layer
            rows = self.kernel_config.max_clusters
            self._centroids = [tuple(torch.zeros((batch * self.h_kv, rows, 128), dtype=torch.float16, device=self.device)
                                     for _ in range(2)) for _ in self.caches]
            self._sync_graph_inputs()
            # scratch for any compressed length up to 2^20 tokens with the library's own schedule
            need = library().reskv_decode_bitmap_fp16_workspace_bytes(batch, self.h_kv, self.h_q, 1 << 20, 0)
            self._workspace = torch.zeros(need, dtype=torch.uint8, device=self.device)
        else:
            if _flash_kvcache is None:
                raise RuntimeError("graph decode of the dense baseline needs flash_attn")
            self._state = torch.tensor([self.length, 0], dtype=torch.int32, device=self.device)
            self._seqlens = torch.full((batch,), self.length, dtype=torch.int32, device=self.device)
            for c in self.caches:  # flash_attn_with_kvcache wants [B, T, H, D]
                c.k = c.k.transpose(1, 2).contiguous()
                c.v = c.v.transpose(1, 2).contiguous()

    def _sync_graph_inputs(self):
        """Refresh what a captured step reads: counts in the step state, centroid tables, and the
        addresses of the compressed buffers (a buffer that had to grow invalidates the graph)."""
        comp = self.caches[0].compressed
        self._state.copy_(torch.tensor([self.length, self.caches[0].live, comp.seq_len if comp is not None else -1, 0],
                                       dtype=torch.int32))
        addresses = []
        for cache, (kc, vc) in zip(self.caches, self._centroids):
            if cache.compressed is None:
                raise RuntimeError("graph decode needs a compressed segment (prompt shorter than recent + group)")
            for table, tensor in ((kc, cache.compressed.key), (vc, cache.compressed.value)):
                native = tensor._native
                table[:, :native[0].shape[1]].copy_(native[0])
                addresses += [t.data_ptr() for t in native[1:] if t is not None] + [tensor.token_stride]
        if addresses != getattr(self, "_graph_addresses", None):
            self._graph_addresses = addresses
            self._graph = None

    @torch.no_grad()
    def decode_graph(self, tokens: torch.Tensor) -> torch.Tensor:
        """Same result as ``decode`` but replaying a captured CUDA graph of the step."""
        if self.cache_kind == "reskv" and self.caches[0].live + 1 == self.caches[0].keys.shape[2]:
            # this token fills the window.  The eager step appends it and then compresses the oldest
            # group before attending (as the reference does); the group does not contain the new
            # token, so compressing it first and appending afterwards gives the same cache.  That is
            # done here, outside the graph; the graph then only needs the new counts.
            for cache in self.caches:
                cache._compress_oldest_group()
            self._sync_graph_inputs()
        self._tok_in.copy_(tokens)
        if self._graph is None and not self._warmed:
            # once: a warm-up outside capture (library handles, lazy inits), on a state copy that is restored
            self._warmed = True
            saved = self._state.clone()
            saved_len = None if self.cache_kind == "reskv" else self._seqlens.clone()
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self._step_body(self._tok_in)
            torch.cuda.current_stream(self.device).wait_stream(side)
            self._state.copy_(saved)
            if saved_len is not None:
                self._seqlens.copy_(saved_len)
        if self._graph is None:
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._logits_out = self._step_body(self._tok_in)
        self._graph.replay()
        self.length += 1
        if self.cache_kind == "reskv":
            for cache in self.caches:
                cache.live += 1
                cache.length += 1
        return self._logits_out

    def cache_bytes(self) -> int:
        total = 0
        for c in self.caches or []:
            if isinstance(c, _DenseLayerCache):
                total += c.k.nbytes + c.v.nbytes
            else:
                total += (c.compressed.nbytes if c.compressed is not None else 0)
                total += c.keys.nbytes + c.raw_keys.nbytes + c.values.nbytes
        return total
