"""Weights: names, dtypes, the one error that lists every fault, random folders (no GPU)."""
import json

import pytest
import torch
from safetensors.torch import save_file

from conftest import TINY_CONFIGS, TINY_LLAMA, TINY_QWEN, read_folder
from helios_b200.config import resolve_architecture
from helios_b200.weights import WeightsError, expected_tensors, load_weights, random_tensors


def _plan(raw):
    arch = resolve_architecture(raw)
    return arch.build_plan(arch.parse_config(raw))


def test_expected_names_are_the_checkpoint_names():
    names = set(expected_tensors(_plan(TINY_QWEN)))
    assert "model.embed_tokens.weight" in names and "lm_head.weight" in names
    assert "model.layers.2.self_attn.k_proj.bias" in names
    assert "model.layers.0.mlp.down_proj.weight" in names and "model.norm.weight" in names
    assert not any("bias" in n for n in expected_tensors(_plan(TINY_LLAMA)))


@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_random_folder_round_trip(model_folders, name):
    cfg, tensors = read_folder(model_folders[name])
    assert cfg == TINY_CONFIGS[name]
    plan = _plan(cfg)
    want = {n for n in expected_tensors(plan) if n not in plan.tied}
    assert set(tensors) == want
    assert all(t.dtype == torch.float32 for t in tensors.values())
    # seeded: the same again
    from conftest import TINY_SEEDS
    again = random_tensors(_plan(cfg), TINY_SEEDS[name])
    assert all(torch.equal(again[k], tensors[k]) for k in tensors)
    # norm weights around one, matrices around zero with std 0.02
    assert abs(float(tensors["model.norm.weight"].mean()) - 1.0) < 0.02
    assert 0.015 < float(tensors["model.layers.0.mlp.up_proj.weight"].std()) < 0.025
    load_weights(plan, model_folders[name], torch.bfloat16, "cpu")
    assert plan.layers[0].mixer.w_qkv.dtype == torch.bfloat16
    assert plan.final_norm.weight.dtype == torch.float32
    if cfg["tie_word_embeddings"]:
        assert plan.head.weight.data_ptr() == plan.embedding.table.data_ptr()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_folders, tmp_path):
    cfg, tensors = read_folder(model_folders["tiny_llama"])
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)   # a buffer: fine
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 127)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsError) as exc:
        load_weights(_plan(cfg), tmp_path, torch.float32, "cpu")
    e = exc.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.mlp.down_proj.weight"]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shape", "model.norm.weight", "(64, 127)"):
        assert word in msg


def test_a_qwen_checkpoint_on_a_llama_configuration_is_refused(model_folders, tmp_path):
    # python/helios/exec/loader.py:105-114: biases without a slot must not be dropped silently
    _, tensors = read_folder(model_folders["tiny_qwen"])
    cfg = dict(TINY_QWEN, architectures=["LlamaForCausalLM"], model_type="llama")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsError) as exc:
        load_weights(_plan(cfg), tmp_path, torch.float32, "cpu")
    assert any(n.endswith("q_proj.bias") for n in exc.value.unexpected)


def test_sharded_checkpoint_and_missing_files(model_folders, tmp_path):
    cfg, tensors = read_folder(model_folders["tiny_llama"])
    names = sorted(tensors)
    a, b = names[: len(names) // 2], names[len(names) // 2:]
    save_file({k: tensors[k] for k in a}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in b}, str(tmp_path / "model-00002-of-00002.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        **{k: "model-00001-of-00002.safetensors" for k in a},
        **{k: "model-00002-of-00002.safetensors" for k in b}}}))
    plan = _plan(cfg)
    load_weights(plan, tmp_path, torch.float32, "cpu")
    assert torch.equal(plan.final_norm.weight, tensors["model.norm.weight"])
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError):
        load_weights(_plan(cfg), empty, torch.float32, "cpu")


def test_tied_head_may_also_be_stored(model_folders, tmp_path):
    cfg, tensors = read_folder(model_folders["tiny_qwen"])
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"] * 2
    save_file(tensors, str(tmp_path / "model.safetensors"))
    plan = _plan(cfg)
    load_weights(plan, tmp_path, torch.float32, "cpu")
    assert torch.equal(plan.head.weight, tensors["lm_head.weight"])
