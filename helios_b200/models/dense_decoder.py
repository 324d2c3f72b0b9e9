"""Plan of the dense GQA decoder that ``LlamaForCausalLM`` and ``Qwen2ForCausalLM``
name (python/helios/exec/model.py:395-430): embedding, pre-norm blocks of
grouped-query attention and SwiGLU, final RMSNorm, output head, rotary positions.

The parts are chosen by name from the part registries, layer by layer, so a layer
with a window gets an attention part with that window and the cache manager puts
it into a group of its own.
"""
from __future__ import annotations

from ..config.model_config import DenseDecoderConfig
from ..config.registry import register_architecture
from ..parts import ModelPlan, OutputHead, TokenEmbedding, part_class


def build_dense_decoder_plan(cfg: DenseDecoderConfig) -> ModelPlan:
    norm_cls = part_class("norm", "rmsnorm")
    mixer_cls = part_class("mixer", "gqa_attention")
    ffn_cls = part_class("feed_forward", "swiglu")
    block_cls = part_class("block", "pre_norm")
    rope_cls = part_class("position_encoding", "rotary")

    rope = rope_cls(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling)
    layers, prefixes = [], []
    for i in range(cfg.num_hidden_layers):
        layers.append(block_cls(
            norm_cls(cfg.hidden_size, cfg.rms_norm_eps),
            mixer_cls(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                      cfg.head_dim, cfg.attention_scale, cfg.attention_bias,
                      window=cfg.layer_windows[i], position=rope),
            norm_cls(cfg.hidden_size, cfg.rms_norm_eps),
            ffn_cls(cfg.hidden_size, cfg.intermediate_size),
        ))
        prefixes.append(f"model.layers.{i}.")
    tied = {"lm_head.weight": "model.embed_tokens.weight"} if cfg.tie_word_embeddings else {}
    plan = ModelPlan(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab_size, cfg.hidden_size),
        position=rope,
        layers=layers,
        layer_prefixes=prefixes,
        final_norm=norm_cls(cfg.hidden_size, cfg.rms_norm_eps),
        head=OutputHead(cfg.vocab_size, cfg.hidden_size),
        tied=tied,
    )
    return plan


def _toy_config(architecture: str, model_type: str):
    """config.json for a small model of this family from the sizes ``make-toy-model`` takes
    (python/helios/cli.py:161-179 builds the reference's one toy configuration)."""
    def toy(sizes):
        hidden = sizes["hidden_size"]
        cfg = {
            "architectures": [architecture], "model_type": model_type,
            "vocab_size": sizes["vocab_size"], "hidden_size": hidden,
            "intermediate_size": sizes.get("intermediate_size") or 2 * hidden,
            "num_hidden_layers": sizes["layers"], "num_attention_heads": sizes["heads"],
            "num_key_value_heads": sizes["kv_heads"], "max_position_embeddings": sizes["max_pos"],
            "rms_norm_eps": sizes["rms_eps"], "rope_theta": sizes["rope_theta"],
            "tie_word_embeddings": bool(sizes.get("tie")), "hidden_act": "silu",
            "torch_dtype": "float32", "attention_bias": model_type == "qwen2",
            "bos_token_id": 1, "eos_token_id": 2,
        }
        if sizes.get("head_dim"):
            cfg["head_dim"] = sizes["head_dim"]
        if sizes.get("rope_scaling"):
            f, lo, hi, orig = sizes["rope_scaling"]
            cfg["rope_scaling"] = {"rope_type": "llama3", "factor": f, "low_freq_factor": lo,
                                   "high_freq_factor": hi,
                                   "original_max_position_embeddings": int(orig)}
        if sizes.get("sliding_window"):
            cfg.update(sliding_window=sizes["sliding_window"], use_sliding_window=True,
                       max_window_layers=sizes.get("max_window_layers") or 0)
        return cfg
    return toy


def _parse(architecture: str):
    def parse(cfg_dict):
        return DenseDecoderConfig.from_hf(cfg_dict, architecture=architecture)
    return parse


for _name, _type in (("LlamaForCausalLM", "llama"), ("Qwen2ForCausalLM", "qwen2")):
    register_architecture(_name, _parse(_name), build_dense_decoder_plan,
                          toy_config=_toy_config(_name, _type), replace=True)
