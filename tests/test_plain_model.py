"""The plain implementation itself (no GPU): against the reference's stored logits, and
each of its parts against a hand calculation."""
import math
from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

import plain_model
from golden.make_golden import GOLDEN_CONFIGS, golden_inputs

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", list(GOLDEN_CONFIGS))
def test_plain_matches_the_reference_models_logits(name):
    cfg, weights, tokens = golden_inputs(name)
    stored = load_file(str(GOLDEN / f"golden_{name}.safetensors"))
    assert stored["tokens"].tolist() == tokens, "the seeded inputs changed; run make_golden.py again"
    plain = plain_model.forward_logits(cfg, weights, tokens)
    assert (plain - stored["logits"].double()).abs().max().item() < 1e-5


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    out = plain_model.rms_norm(x, w, 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]], dtype=torch.float64))


def test_llama3_scaling_by_hand():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = plain_model.rope_inv_freq(16, 500000.0, None)
    got = plain_model.rope_inv_freq(16, 500000.0, sc)
    for j in range(8):
        wl = 2 * math.pi / float(base[j])
        if wl < 64 / 4:
            want = float(base[j])
        elif wl > 64 / 1:
            want = float(base[j]) / 8
        else:
            s = (64 / wl - 1.0) / 3.0
            want = (1 - s) * float(base[j]) / 8 + s * float(base[j])
        assert float(got[j]) == pytest.approx(want, rel=1e-12)
    kinds = [2 * math.pi / float(b) for b in base]
    assert any(k < 16 for k in kinds) and any(k > 64 for k in kinds) and any(16 <= k <= 64 for k in kinds)


def test_rope_is_a_rotation_of_half_pairs():
    x = torch.zeros(1, 1, 4, dtype=torch.float64)
    x[0, 0, 0] = 1.0                       # pair (0, 2)
    inv = torch.tensor([1.0, 0.0], dtype=torch.float64)
    out = plain_model.apply_rope(x, torch.tensor([1]), inv)
    assert torch.allclose(out[0, 0], torch.tensor([math.cos(1), 0, math.sin(1), 0], dtype=torch.float64))


def test_attention_mask_and_window():
    n, hd = 6, 4
    q = torch.zeros(n, 1, hd, dtype=torch.float64)
    k = torch.zeros(n, 1, hd, dtype=torch.float64)
    v = torch.arange(n, dtype=torch.float64)[:, None, None].expand(n, 1, hd).clone()
    out = plain_model.causal_attention(q, k, v, 1.0, None)          # uniform over 0..i
    assert torch.allclose(out[:, 0, 0], torch.tensor([0, .5, 1, 1.5, 2, 2.5], dtype=torch.float64))
    out = plain_model.causal_attention(q, k, v, 1.0, 2)             # uniform over i-1..i
    assert torch.allclose(out[:, 0, 0], torch.tensor([0, .5, 1.5, 2.5, 3.5, 4.5], dtype=torch.float64))


def test_gqa_head_mapping():
    # query heads 0,1 read KV head 0; 2,3 read KV head 1 (python/helios/exec/paged_attn.py:248-261)
    q = torch.zeros(1, 4, 2, dtype=torch.float64)
    k = torch.zeros(1, 2, 2, dtype=torch.float64)
    v = torch.tensor([[[1.0, 1.0], [2.0, 2.0]]], dtype=torch.float64)
    out = plain_model.causal_attention(q, k, v, 1.0, None)
    assert out[0, :, 0].tolist() == [1.0, 1.0, 2.0, 2.0]


def test_layer_windows_and_bias_rules():
    cfg = {"num_hidden_layers": 4, "sliding_window": 9, "use_sliding_window": True, "max_window_layers": 2}
    assert plain_model.layer_windows(cfg) == [None, None, 9, 9]
    assert plain_model.layer_windows(dict(cfg, use_sliding_window=False)) == [None] * 4
    assert plain_model.has_qkv_bias({"model_type": "qwen2"}) and not plain_model.has_qkv_bias({"model_type": "llama"})
    assert not plain_model.has_qkv_bias({"model_type": "qwen2", "attention_bias": False})


def test_sampling_reference_rules():
    logits = torch.tensor([0.0, 1.0, 2.0, 3.0])
    assert plain_model.sample_reference(logits, 1.0, 1, 1.0, 0.999) == 3         # top-1
    assert plain_model.sample_reference(logits, 1.0, 0, 0.5, 0.999) == 3         # 0.64 crosses 0.5 alone
    assert plain_model.sample_reference(logits, 1.0, 0, 0.7, 0.999) == 3         # index order: 2 then 3
    assert plain_model.sample_reference(logits, 1.0, 0, 0.7, 0.0) == 2
    assert plain_model.sample_reference(logits, 1.0, 0, 1.0, 0.0) == 0
