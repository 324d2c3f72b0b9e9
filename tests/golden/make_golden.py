"""Compares the plain implementation (tests/plain_model.py) with the reference's own
model code, once, on the CPU, and stores the reference's logits.

    python tests/golden/make_golden.py --reference /path/to/helios/python

The reference's ``HeliosModel`` (python/helios/exec/model.py) is imported from the
given path, filled with this repository's seeded random weights by name (its
parameter names are the checkpoint names without ``model.``,
python/helios/exec/loader.py:170-176), and run whole over a seeded token sequence with
``forward_all_logits`` (model.py:498-521) over an identity block table.  Only
what the reference can express is covered: no rope scaling, no explicit head_dim,
no window.  The outputs, ``golden_<name>.safetensors`` (tokens, float32 logits),
are committed; tests/test_plain_model.py checks the plain implementation against
them without needing the reference.
"""
import argparse
import sys
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

GOLDEN_CONFIGS = {
    # tiny Llama sizes without the scaling the reference lacks
    "llama": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 256,
        "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 256,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "attention_bias": False,
        "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "float32",
    },
    # tiny Qwen sizes: bias, one KV head, tied head
    "qwen": {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 384,
        "hidden_size": 96, "intermediate_size": 224, "num_hidden_layers": 3,
        "num_attention_heads": 6, "num_key_value_heads": 1, "max_position_embeddings": 512,
        "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True,
        "hidden_act": "silu", "torch_dtype": "float32",
    },
}
GOLDEN_SEEDS = {"llama": 5, "qwen": 6}
GOLDEN_TOKENS = 37


def golden_inputs(name):
    from helios_b200.config import resolve_architecture
    from helios_b200.weights import random_tensors

    cfg = GOLDEN_CONFIGS[name]
    arch = resolve_architecture(cfg)
    plan = arch.build_plan(arch.parse_config(cfg))
    weights = random_tensors(plan, GOLDEN_SEEDS[name])
    g = torch.Generator().manual_seed(GOLDEN_SEEDS[name] + 100)
    tokens = torch.randint(0, cfg["vocab_size"], (GOLDEN_TOKENS,), generator=g).tolist()
    return cfg, weights, tokens


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="the reference's python/ folder")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from helios.exec.model import HeliosModel, ModelConfig
    from helios.exec.paged_attn import PagedKVCache
    import plain_model

    for name in GOLDEN_CONFIGS:
        cfg, weights, tokens = golden_inputs(name)
        mc = ModelConfig.from_hf(cfg)
        model = HeliosModel(mc).to(torch.float32).eval()
        own = dict(model.named_parameters())
        with torch.no_grad():
            for key, t in weights.items():
                own[key if key.startswith("lm_head.") else key[len("model."):]].copy_(t)
            if cfg["tie_word_embeddings"]:
                model.lm_head.weight.copy_(model.embed_tokens.weight)
        n, bs = len(tokens), 4
        blocks = list(range((n + bs - 1) // bs))
        caches = [PagedKVCache(len(blocks), bs, mc.num_key_value_heads, mc.head_dim)
                  for _ in range(mc.num_hidden_layers)]
        with torch.no_grad():
            ref = model.forward_all_logits(tokens, list(range(n)), caches, blocks, n)
        plain = plain_model.forward_logits(cfg, weights, tokens)
        err = (ref.double() - plain).abs().max().item()
        print(f"{name}: reference vs plain max |err| = {err:.3e}")
        assert err < 1e-5
        save_file({"tokens": torch.tensor(tokens, dtype=torch.int32), "logits": ref.contiguous()},
                  str(HERE / f"golden_{name}.safetensors"))


if __name__ == "__main__":
    main()
