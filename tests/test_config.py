"""Configuration and registry (no GPU)."""
import copy

import pytest

from conftest import TINY_CONFIGS, TINY_LLAMA, TINY_QWEN, TINY_TILED, TINY_WINDOW
from helios_b200.config import (ConfigError, DenseDecoderConfig, known_architectures,
                                register_architecture, resolve_architecture,
                                unregister_architecture)


def test_registry_knows_both_names_and_lists_them_on_error():
    assert {"LlamaForCausalLM", "Qwen2ForCausalLM"} <= set(known_architectures())
    with pytest.raises(ConfigError) as exc:
        resolve_architecture({"architectures": ["MambaForCausalLM"]})
    assert "LlamaForCausalLM" in str(exc.value) and "MambaForCausalLM" in str(exc.value)
    with pytest.raises(ConfigError):
        resolve_architecture({})


@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_every_key_is_read(name):
    raw = TINY_CONFIGS[name]
    cfg = resolve_architecture(raw).parse_config(raw)
    assert cfg.vocab_size == raw["vocab_size"]
    assert cfg.hidden_size == raw["hidden_size"]
    assert cfg.intermediate_size == raw["intermediate_size"]
    assert cfg.num_hidden_layers == raw["num_hidden_layers"]
    assert cfg.num_attention_heads == raw["num_attention_heads"]
    assert cfg.num_key_value_heads == raw["num_key_value_heads"]
    assert cfg.head_dim == raw.get("head_dim", raw["hidden_size"] // raw["num_attention_heads"])
    assert cfg.rms_norm_eps == raw["rms_norm_eps"]
    assert cfg.rope_theta == raw["rope_theta"]
    assert cfg.tie_word_embeddings == raw["tie_word_embeddings"]
    assert cfg.max_position_embeddings == raw["max_position_embeddings"]
    # and it survives a round trip through config.json
    again = DenseDecoderConfig.from_hf(cfg.to_hf())
    assert again == cfg


def test_defaults_follow_the_reference():
    # python/helios/exec/model.py:60-77
    raw = {"architectures": ["LlamaForCausalLM"], "vocab_size": 10, "hidden_size": 8,
           "intermediate_size": 16, "num_hidden_layers": 1, "num_attention_heads": 2}
    cfg = DenseDecoderConfig.from_hf(raw)
    assert cfg.num_key_value_heads == 2 and cfg.head_dim == 4
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0
    assert cfg.max_position_embeddings == 4096 and not cfg.tie_word_embeddings
    assert not cfg.attention_bias and cfg.rope_scaling is None


def test_bias_is_inferred_for_qwen2_and_explicit_key_wins():
    # python/helios/exec/model.py:79-92
    assert DenseDecoderConfig.from_hf(TINY_QWEN).attention_bias
    assert not DenseDecoderConfig.from_hf(TINY_LLAMA).attention_bias
    raw = dict(TINY_QWEN, attention_bias=False)
    assert not DenseDecoderConfig.from_hf(raw).attention_bias
    raw = {k: v for k, v in TINY_LLAMA.items() if k != "attention_bias"}
    raw["architectures"] = ["Qwen2ForCausalLM"]
    assert DenseDecoderConfig.from_hf(raw).attention_bias


def test_rope_scaling_and_windows():
    cfg = DenseDecoderConfig.from_hf(TINY_LLAMA)
    assert cfg.rope_scaling.factor == 8.0 and cfg.rope_scaling.original_max_position_embeddings == 64
    assert DenseDecoderConfig.from_hf(TINY_QWEN).layer_windows == (None, None, None)
    assert DenseDecoderConfig.from_hf(TINY_WINDOW).layer_windows == (None, 40, 40, 40)
    raw = dict(TINY_WINDOW, layer_types=["sliding_attention", "full_attention"] * 2)
    assert DenseDecoderConfig.from_hf(raw).layer_windows == (40, None, 40, None)


def test_a_llama_configuration_with_a_window_is_refused():
    for change in ({"sliding_window": 8, "layer_types": ["sliding_attention", "full_attention"]},
                   {"sliding_window": 8, "use_sliding_window": True, "max_window_layers": 0}):
        with pytest.raises(ConfigError) as exc:
            DenseDecoderConfig.from_hf(dict(TINY_LLAMA, **change))
        assert "LlamaForCausalLM" in str(exc.value)
    # keys that are present but switch nothing on are fine, as in Qwen2.5's own files
    DenseDecoderConfig.from_hf(dict(TINY_LLAMA, sliding_window=8, use_sliding_window=False))
    DenseDecoderConfig.from_hf(dict(TINY_LLAMA, sliding_window=8, layer_types=["full_attention"] * 2))


@pytest.mark.parametrize("change, word", [
    ({"vocab_size": None}, "vocab_size"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"head_dim": 15}, "head_dim"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
])
def test_errors_name_the_key(change, word):
    raw = copy.deepcopy(TINY_LLAMA)
    for k, v in change.items():
        if v is None and k == "vocab_size":
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError) as exc:
        DenseDecoderConfig.from_hf(raw)
    assert word in str(exc.value)


def test_a_test_can_register_an_architecture():
    register_architecture("ToyForCausalLM", lambda d: d, lambda c: None)
    try:
        assert resolve_architecture({"architectures": ["ToyForCausalLM"]}).name == "ToyForCausalLM"
        with pytest.raises(ValueError):
            register_architecture("ToyForCausalLM", lambda d: d, lambda c: None)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_plan_takes_every_size_from_the_configuration():
    from helios_b200.models import build_dense_decoder_plan

    for raw in TINY_CONFIGS.values():
        cfg = DenseDecoderConfig.from_hf(raw)
        plan = build_dense_decoder_plan(cfg)
        assert len(plan.layers) == cfg.num_hidden_layers
        assert [r.layer for r in plan.schedule] == list(range(cfg.num_hidden_layers))
        for i, block in enumerate(plan.layers):
            m = block.mixer
            assert (m.num_heads, m.num_kv_heads, m.head_dim) == (
                cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim)
            assert m.window == cfg.layer_windows[i] and m.qkv_bias == cfg.attention_bias
            assert m.scale == pytest.approx(cfg.head_dim ** -0.5)
            assert block.mixer_norm.eps == cfg.rms_norm_eps
            assert block.ffn.inner == cfg.intermediate_size


def test_a_plan_names_the_kernel_libraries_its_sizes_need():
    """What a model compiles when it is made follows its parts' sizes and the dtype: heads of
    16 have no tiled attention kernel, heads of 32 no tcgen05 one, float32 neither."""
    import torch
    from helios_b200.csrc.build import LIBRARIES
    from helios_b200.models import build_dense_decoder_plan

    def libraries(raw, dtype):
        plan = build_dense_decoder_plan(DenseDecoderConfig.from_hf(raw))
        return {n for _p, part in plan.named_parts() for n in part.kernel_libraries(dtype)}

    bf16, f32 = torch.bfloat16, torch.float32
    assert libraries(TINY_LLAMA, bf16) == {"gemm_bf16", "attention_generic"}
    assert libraries(TINY_TILED, bf16) == {"gemm_bf16", "attention_bf16"}
    assert libraries(TINY_TILED, f32) == {"gemm_f32", "attention_generic"}
    wide = dict(TINY_LLAMA, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8)
    assert libraries(wide, bf16) == {"gemm_bf16", "attention_bf16", "attention_tc", "attention_pair"}
    for raw in TINY_CONFIGS.values():
        assert libraries(raw, bf16) | libraries(raw, f32) <= set(LIBRARIES)
