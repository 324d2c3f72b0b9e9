"""Random weights from a configuration and a seed
(python/helios/exec/loader.py:179-231, ``save_toy_model``).

``write_model_folder`` writes ``config.json`` and ``model.safetensors`` (float32)
for any configuration of a registered architecture, plus a byte-level tokenizer;
``bind_random_weights`` fills a plan on the device without a file, for sizes
where writing one would be wasteful.  Matrices are N(0, 0.02), norm weights
1 + N(0, 0.02), biases N(0, 0.02).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict

import torch

from ..config.registry import resolve_architecture
from ..parts import ModelPlan, WeightSpec
from .loader import bind_tensors, expected_tensors, target_dtype


def _draw(spec: WeightSpec, gen: torch.Generator, device) -> torch.Tensor:
    if spec.init == "normal":
        return torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32) * spec.std
    if spec.init == "ones_jitter":
        return 1.0 + torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32) * spec.std
    if spec.init == "ones":
        return torch.ones(spec.shape, device=device, dtype=torch.float32)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, device=device, dtype=torch.float32)
    raise ValueError(f"unknown init {spec.init!r}")


def random_tensors(plan: ModelPlan, seed: int) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (float32, CPU) in the plan's order; tied names are left out."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name, (_part, _local, spec) in expected_tensors(plan).items():
        if name in plan.tied:
            continue
        t = _draw(spec, gen, "cpu")
        out[name] = t.to(torch.int32) if spec.kind == "table" else t
    return out


def bind_random_weights(plan: ModelPlan, seed: int, compute_dtype: torch.dtype, device) -> None:
    """Draw every tensor on ``device`` and hand it to its part, without a file."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    tensors: Dict[str, torch.Tensor] = {}
    for name, (_part, _local, spec) in expected_tensors(plan).items():
        if name in plan.tied:
            continue
        tensors[name] = _draw(spec, gen, device).to(target_dtype(spec, compute_dtype))
    bind_tensors(plan, tensors)


def write_model_folder(out_dir, config_json: Dict[str, Any], seed: int,
                       tokenizer: bool = True) -> Path:
    """A model folder for the ``config.json`` dictionary ``config_json``."""
    from safetensors.torch import save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    arch = resolve_architecture(config_json)
    cfg = arch.parse_config(config_json)
    plan = arch.build_plan(cfg)
    save_file(random_tensors(plan, seed), str(out / "model.safetensors"))
    with open(out / "config.json", "w", encoding="utf-8") as f:
        json.dump(config_json, f, indent=2)
    if tokenizer:
        write_byte_tokenizer(out, int(config_json["vocab_size"]))
    return out


def write_byte_tokenizer(out: Path, vocab_size: int) -> None:
    """A byte-level vocabulary, so that a random model folder takes text prompts without
    any download (the idea of python/helios/exec/loader.py:234-301).  Ids 0..2 are
    <pad>, <s>, </s>; byte b is id 3 + b as far as the vocabulary reaches."""
    with open(out / "byte_tokenizer.json", "w", encoding="utf-8") as f:
        json.dump({"type": "helios_b200.byte", "vocab_size": vocab_size, "pad": 0, "bos": 1,
                   "eos": 2, "first_byte_id": 3}, f, indent=2)
