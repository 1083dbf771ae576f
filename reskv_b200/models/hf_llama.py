"""Hugging Face Llama checkpoints on the compressed KV cache.

``ResKVForCausalLM`` is a ``LlamaForCausalLM`` whose attention layers keep a
``ResKVCache``: prefill attends densely and then compresses, every later token
is attended through the fused compressed-cache kernels.  Same contract as the
reference class of that name (reskv/models/llama.py:25-170): FP16 CUDA
inference, 128-wide heads, GQA ratios 1 / 4 / 8, equal-length unpadded batches,
one new token per continuation step, positions contiguous from zero, last-token
logits by default.  Written against the ``transformers`` 5.x module interfaces.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from transformers import LlamaForCausalLM
from transformers.models.llama.modeling_llama import LlamaAttention, LlamaMLP, apply_rotary_pos_emb

from .._attention import attention
from ..cache import ResKVCache
from ..config import ResKVKernelConfig, _model_settings

_SUPPORTED_ROPE = ("default", "llama3", "linear")


class ResKVMLP(LlamaMLP):
    """Feed-forward block for inference: the up projection is multiplied into the activated gate in place, so
    one ``[..., intermediate]`` temporary lives at a time instead of two (same role as the reference's class
    of this name, reskv/models/llama.py:14-22).  Whenever autograd is recording, or in training mode, it is the
    stock ``LlamaMLP`` -- the in-place product would destroy a tensor the backward pass needs."""

    def forward(self, x):
        if self.training or torch.is_grad_enabled():
            return super().forward(x)
        hidden = self.act_fn(self.gate_proj(x))
        hidden *= self.up_proj(x)
        return self.down_proj(hidden)


class ResKVAttention(LlamaAttention):
    """Attention layer that reads and feeds one ``ResKVLayerCache``."""

    rope_frequencies: torch.Tensor | None = None  # FP32 [64], set by the model before every forward

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, **kwargs):
        lead = hidden_states.shape[:-1]  # (batch, tokens)
        split = (*lead, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(split).transpose(1, 2)
        k = self.k_proj(hidden_states).view(split).transpose(1, 2)
        v = self.v_proj(hidden_states).view(split).transpose(1, 2)
        cos, sin = position_embeddings
        q_rot, k_rot = apply_rotary_pos_emb(q, k, cos, sin)
        layer = None if past_key_values is None else past_key_values.layers[self.layer_idx]
        if layer is not None and layer.length > 0:
            # continuation: the cache takes the token (compressing the oldest group when the
            # window is full) and the fused kernels attend over compressed + dense segments
            if lead[1] != 1:
                raise ValueError("only single-token continuation is supported")
            window_k, window_v = layer.update(k_rot, v, {"raw_keys": k})
            if layer.compressed is None:
                out = F.scaled_dot_product_attention(q_rot, window_k, window_v, enable_gqa=True, scale=self.scaling)
            else:
                model_rope = layer.config.rope_mode == "model"
                out = attention(q, layer.compressed, position=layer.length - 1,
                                start_position=layer.start_position, rope_theta=_rope_theta(self.config),
                                inv_freq=self.rope_frequencies if model_rope else None,
                                scaling=self.scaling, recent=(q_rot, window_k, window_v))
        else:
            # prompt: dense attention first, compression afterwards
            out = F.scaled_dot_product_attention(q_rot, k_rot, v, attn_mask=attention_mask,
                                                 is_causal=attention_mask is None and lead[1] > 1,
                                                 enable_gqa=True, scale=self.scaling)
            if layer is not None:
                layer.update(k_rot, v, {"raw_keys": k})
        return self.o_proj(out.transpose(1, 2).reshape(*lead, -1).contiguous()), None


def _rope_theta(config) -> float:
    params = getattr(config, "rope_parameters", None) or {}
    return float(params.get("rope_theta", getattr(config, "rope_theta", 500000.0)))


def _rope_type(config) -> str:
    params = getattr(config, "rope_parameters", None) or getattr(config, "rope_scaling", None) or {}
    return params.get("rope_type", "default")


class ResKVForCausalLM(LlamaForCausalLM):
    """``LlamaForCausalLM`` with the compressed KV cache; settings travel in
    ``config.reskv_kernel_config`` so that ``save_pretrained`` / ``from_pretrained`` keep them."""

    def __init__(self, config, kernel_config: ResKVKernelConfig | None = None):
        if config.model_type != "llama":
            raise ValueError("ResKV CUDA inference requires a Llama configuration")
        settings = _model_settings(config, kernel_config, ResKVKernelConfig, "reskv_kernel_config")
        head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        if head_dim != 128:
            raise ValueError("ResKV requires head_dim=128")
        kv, heads = config.num_key_value_heads, config.num_attention_heads
        if kv < 1 or heads % kv:
            raise ValueError("query heads must be a positive integer multiple of KV heads")
        if heads // kv not in (1, 4, 8):
            raise ValueError("ResKV supports GQA ratios 1, 4, and 8")
        if settings.rope_mode == "model" and _rope_type(config) not in _SUPPORTED_ROPE:
            raise ValueError("this release supports static default, llama3, and linear RoPE")
        config._attn_implementation = "sdpa"
        super().__init__(config)
        self.kernel_config = settings
        for index, block in enumerate(self.model.layers):
            block.self_attn = ResKVAttention(config, index)
            block.mlp = ResKVMLP(config)
        self.post_init()

    @classmethod
    def _supports_default_dynamic_cache(cls):
        return False

    def _frequencies(self) -> torch.Tensor:
        """FP32 rotary frequencies; recomputed when ``.half()`` has rounded the buffer."""
        rotary = self.model.rotary_emb
        freq = rotary.inv_freq
        if freq.dtype != torch.float32:
            init = getattr(rotary, "rope_init_fn", None)
            if init is not None:
                freq, rotary.attention_scaling = init(self.config, device=torch.device("cpu"))
            else:
                half = torch.arange(0, 128, 2, dtype=torch.float32) / 128
                freq = _rope_theta(self.config) ** -half
            freq = freq.float().to(rotary.inv_freq.device)
            rotary.register_buffer("inv_freq", freq, persistent=False)
            rotary.original_inv_freq = freq
        return freq

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                inputs_embeds=None, labels=None, use_cache=None, cache_position=None, logits_to_keep=1, **kwargs):
        use_cache = self.config.use_cache if use_cache is None else use_cache
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("provide exactly one of input_ids or inputs_embeds")
        if labels is not None or self.training:
            raise ValueError("ResKV is an inference implementation; call model.eval()")
        if past_key_values is not None and not isinstance(past_key_values, ResKVCache):
            raise ValueError("past_key_values must be a ResKVCache")
        if use_cache and past_key_values is None:
            # `sink_tokens` (default 0, like the reference's CUDA cache) may be set on the model instance
            past_key_values = ResKVCache(self.kernel_config, len(self.model.layers), getattr(self, "sink_tokens", 0))
        if attention_mask is not None and not bool(attention_mask.eq(1).all()):
            raise ValueError("ResKV requires equal-length unpadded batches")
        given = input_ids if input_ids is not None else inputs_embeds
        length = given.shape[1]
        seen = 0 if past_key_values is None else past_key_values.get_seq_length()
        expected = torch.arange(seen, seen + length, device=given.device)
        for positions in (position_ids, cache_position):
            if positions is not None and (positions.device != given.device or not bool(positions.eq(expected).all())):
                raise ValueError("ResKV positions must be contiguous and start at zero")
        freq = self._frequencies() if self.kernel_config.rope_mode == "model" else None
        for block in self.model.layers:
            block.self_attn.rope_frequencies = freq
        extra = {} if cache_position is None else {"cache_position": cache_position}
        return super().forward(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                               past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache,
                               logits_to_keep=logits_to_keep, **extra, **kwargs)
