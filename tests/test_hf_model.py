"""``ResKVForCausalLM`` (Hugging Face Llama on the compressed cache): argument checks on CPU, and on
the GPU the same weights in the Hugging Face wrapper and in the self-contained ``ResKVLlama`` must
give the same logits through prefill, dense-window steps and group compressions."""

import pytest
import torch

transformers = pytest.importorskip("transformers")

TINY = dict(hidden=512, layers=2, heads=4, kv_heads=1, ffn=1024, vocab=320)


def _hf_config():
    from transformers import LlamaConfig

    return LlamaConfig(hidden_size=TINY["hidden"], num_attention_heads=TINY["heads"], num_key_value_heads=TINY["kv_heads"],
                       num_hidden_layers=TINY["layers"], intermediate_size=TINY["ffn"], vocab_size=TINY["vocab"],
                       rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=4096, tie_word_embeddings=False,
                       attention_bias=False, mlp_bias=False)


def _settings():
    from reskv_b200 import ResKVKernelConfig

    return ResKVKernelConfig(sparsity=0.75, layout="unstructured", num_clusters=4, max_clusters=8, group_size=16,
                             recent_size=8, kmeans_iterations=3)


def test_configuration_checks():
    from transformers import LlamaConfig

    from reskv_b200 import ResKVConfig
    from reskv_b200.models import ResKVForCausalLM

    base = dict(hidden_size=512, num_attention_heads=4, num_key_value_heads=1, num_hidden_layers=1, intermediate_size=64,
                vocab_size=32)
    with pytest.raises(ValueError, match="head_dim=128"):
        ResKVForCausalLM(LlamaConfig(**{**base, "num_attention_heads": 8}))
    with pytest.raises(ValueError, match="GQA ratios"):
        ResKVForCausalLM(LlamaConfig(**{**base, "num_key_value_heads": 2}))
    with pytest.raises(TypeError, match="ResKVKernelConfig"):
        ResKVForCausalLM(LlamaConfig(**base), ResKVConfig())
    model = ResKVForCausalLM(LlamaConfig(**base), _settings()).eval()
    assert model.config.reskv_kernel_config["group_size"] == 16  # travels with save_pretrained
    assert type(model.model.layers[0].self_attn).__name__ == "ResKVAttention"
    ids = torch.zeros((1, 3), dtype=torch.long)
    with pytest.raises(ValueError, match="exactly one"):
        model(input_ids=ids, inputs_embeds=torch.zeros(1, 3, 512))
    with pytest.raises(ValueError, match="unpadded"):
        model(input_ids=ids, attention_mask=torch.tensor([[0, 1, 1]]))
    with pytest.raises(ValueError, match="ResKVCache"):
        model(input_ids=ids, past_key_values=transformers.DynamicCache())
    with pytest.raises(ValueError, match="contiguous"):
        model(input_ids=ids, position_ids=torch.tensor([[1, 2, 3]]))
    with pytest.raises(ValueError, match="inference"):
        model(input_ids=ids, labels=ids)


def _load_same_weights(hf, plain):
    """Copy the plain-tensor model's weights into the Hugging Face module tree."""
    hq, hkv = plain.h_q * 128, plain.h_kv * 128
    state = {"model.embed_tokens.weight": plain.embed, "lm_head.weight": plain.lm_head,
             "model.norm.weight": plain.final_norm}
    for i, layer in enumerate(plain.layers):
        pre = f"model.layers.{i}."
        wq, wk, wv = layer["wqkv"].split((hq, hkv, hkv))
        gate, up = layer["w_gate_up"].split((plain.ffn, plain.ffn))
        state.update({pre + "self_attn.q_proj.weight": wq, pre + "self_attn.k_proj.weight": wk,
                      pre + "self_attn.v_proj.weight": wv, pre + "self_attn.o_proj.weight": layer["wo"],
                      pre + "mlp.gate_proj.weight": gate, pre + "mlp.up_proj.weight": up,
                      pre + "mlp.down_proj.weight": layer["w_down"], pre + "input_layernorm.weight": layer["norm1"],
                      pre + "post_attention_layernorm.weight": layer["norm2"]})
    missing, unexpected = hf.load_state_dict(state, strict=False)
    assert not unexpected and all("rotary" in name or "inv_freq" in name for name in missing), (missing, unexpected)


@pytest.mark.gpu
def test_same_logits_as_the_self_contained_model():
    from reskv_b200.cache import ResKVCache
    from reskv_b200.models import LlamaShape, ResKVForCausalLM, ResKVLlama

    cfg = _settings()
    plain = ResKVLlama(LlamaShape(**TINY), cfg, seed=5)
    hf = ResKVForCausalLM(_hf_config(), cfg).half().cuda().eval()
    _load_same_weights(hf, plain)
    ids = torch.randint(0, 320, (2, 70), generator=torch.Generator().manual_seed(1)).cuda()
    cache = ResKVCache(cfg, TINY["layers"])
    with torch.no_grad():
        want = plain.prefill(ids)
        got = hf(input_ids=ids, past_key_values=cache, use_cache=True).logits[:, -1].float()
        torch.testing.assert_close(got, want, atol=3e-2, rtol=3e-2)
        tok = want.argmax(-1)
        for step in range(40):  # crosses two group compressions
            want = plain.decode(tok)
            got = hf(input_ids=tok[:, None], past_key_values=cache, use_cache=True).logits[:, -1].float()
            torch.testing.assert_close(got, want, atol=3e-2, rtol=3e-2)
            tok = want.argmax(-1)
    assert cache.get_seq_length() == plain.length == 110
    assert cache.layers[0].compressed.seq_len == plain.caches[0].compressed.seq_len


@pytest.mark.gpu
def test_generate_runs_on_the_compressed_cache():
    from reskv_b200.cache import ResKVCache
    from reskv_b200.models import ResKVForCausalLM

    cfg = _settings()
    torch.manual_seed(0)
    hf = ResKVForCausalLM(_hf_config(), cfg).half().cuda().eval()
    ids = torch.randint(0, 320, (2, 50), generator=torch.Generator().manual_seed(2)).cuda()
    cache = ResKVCache(cfg, TINY["layers"])
    out = hf.generate(ids, max_new_tokens=30, do_sample=False, past_key_values=cache, pad_token_id=0)
    assert out.shape == (2, 80) and torch.equal(out[:, :50], ids)
    assert cache.layers[0].compressed is not None and cache.get_seq_length() == 79
