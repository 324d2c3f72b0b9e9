"""Shared fixtures: tiny configurations of the architecture that differ in every
size and option, model folders with random weights in a temporary place, and the
tolerances all comparisons use."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Llama-3 style: 2 layers, GQA 4/2, llama3 rope scaling, no bias, untied.
TINY_LLAMA = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "attention_bias": False, "tie_word_embeddings": False, "hidden_act": "silu",
    "torch_dtype": "float32",
}
# Qwen2.5 style: 3 layers, 6 heads on 1 KV head, bias (inferred), tied, window keys present but off.
TINY_QWEN = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 224, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 1, "max_position_embeddings": 512,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True,
    "sliding_window": 128, "use_sliding_window": False, "max_window_layers": 2,
    "hidden_act": "silu", "torch_dtype": "float32",
}
# Qwen2 style with the window on from layer 1, an explicit head_dim that is not width/heads,
# sizes that are no power of two, 5 heads on 5 KV heads.
TINY_WINDOW = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 331, "hidden_size": 80, "intermediate_size": 176, "num_hidden_layers": 4,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "max_position_embeddings": 1024, "rms_norm_eps": 3e-6, "rope_theta": 10000.0,
    "tie_word_embeddings": False, "attention_bias": True,
    "sliding_window": 40, "use_sliding_window": True, "max_window_layers": 1,
    "hidden_act": "silu", "torch_dtype": "float32",
}
# Head sizes the tensor-core attention kernels take (32), GQA 6/2, a window on every
# second layer by an explicit layer_types list, other scaling constants, no bias although Qwen2.
TINY_TILED = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 270, "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32,
    "max_position_embeddings": 2048, "rms_norm_eps": 2e-5, "rope_theta": 10000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 2.0, "original_max_position_embeddings": 32},
    "attention_bias": False, "tie_word_embeddings": True, "hidden_act": "silu",
    "sliding_window": 70, "layer_types": ["full_attention", "sliding_attention", "full_attention"],
    "torch_dtype": "float32",
}
TINY_CONFIGS = {"tiny_llama": TINY_LLAMA, "tiny_qwen": TINY_QWEN, "tiny_window": TINY_WINDOW,
                "tiny_tiled": TINY_TILED}
TINY_SEEDS = {"tiny_llama": 11, "tiny_qwen": 22, "tiny_window": 33, "tiny_tiled": 44}

# float32 path against the plain implementation in float64
F32_ATOL = 2e-5
# bfloat16 path against the plain implementation run on the bfloat16-rounded weights:
# |err| <= BF16_RTOL * max|logits of that row| (8 mantissa bits, a few layers deep)
BF16_RTOL = 3e-2


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (random weights)."""
    from helios_b200.weights import write_model_folder

    out = {}
    base = tmp_path_factory.mktemp("models")
    for name, cfg in TINY_CONFIGS.items():
        out[name] = write_model_folder(base / name, cfg, TINY_SEEDS[name])
    return out


def read_folder(folder):
    """(config.json dict, checkpoint tensors) without any product code."""
    from safetensors.torch import load_file

    with open(Path(folder) / "config.json") as f:
        cfg = json.load(f)
    return cfg, load_file(str(Path(folder) / "model.safetensors"))


def bf16_round(weights):
    """What the bfloat16 path keeps of the checkpoint: matrices rounded to bfloat16,
    vectors (norm weights, biases) as stored."""
    return {k: (v.to(torch.bfloat16).to(torch.float32) if v.dim() >= 2 else v)
            for k, v in weights.items()}


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def assert_logits_close(got, want, dtype, what=""):
    """got: float32 [n, V] from the engine; want: float64 [n, V] from the plain model."""
    got = got.detach().double().cpu()
    want = want.double()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = (got - want).abs()
    if dtype == "float32":
        worst = err.max().item()
        assert worst <= F32_ATOL, f"{what}: max |err| {worst:.3e} > {F32_ATOL} at {_where(err)}"
    else:
        scale = want.abs().amax(dim=-1, keepdim=True)
        rel = (err / scale).max().item()
        assert rel <= BF16_RTOL, f"{what}: max |err|/max|logit| {rel:.3e} > {BF16_RTOL} at {_where(err / scale)}"


def _where(err):
    idx = int(err.argmax())
    return f"row {idx // err.shape[-1]}, column {idx % err.shape[-1]}"
