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

    layers, prefixes = [], []
    for i in range(cfg.num_hidden_layers):
        layers.append(block_cls(
            norm_cls(cfg.hidden_size, cfg.rms_norm_eps),
            mixer_cls(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                      cfg.head_dim, cfg.attention_scale, cfg.attention_bias,
                      window=cfg.layer_windows[i]),
            norm_cls(cfg.hidden_size, cfg.rms_norm_eps),
            ffn_cls(cfg.hidden_size, cfg.intermediate_size),
        ))
        prefixes.append(f"model.layers.{i}.")
    tied = {"lm_head.weight": "model.embed_tokens.weight"} if cfg.tie_word_embeddings else {}
    return ModelPlan(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab_size, cfg.hidden_size),
        position=rope_cls(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling),
        layers=layers,
        layer_prefixes=prefixes,
        final_norm=norm_cls(cfg.hidden_size, cfg.rms_norm_eps),
        head=OutputHead(cfg.vocab_size, cfg.hidden_size),
        tied=tied,
    )


def _parse(architecture: str):
    def parse(cfg_dict):
        return DenseDecoderConfig.from_hf(cfg_dict, architecture=architecture)
    return parse


for _name in ("LlamaForCausalLM", "Qwen2ForCausalLM"):
    register_architecture(_name, _parse(_name), build_dense_decoder_plan, replace=True)
