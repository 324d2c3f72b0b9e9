"""Weights from safetensors, by tensor name
(python/helios/exec/loader.py:43-150).

The plan of the model says which names it expects and with which shapes.  All
faults of a checkpoint are collected and reported in ONE error that lists the
missing tensors, the unexpected ones and those of a wrong shape, so a
half-matching checkpoint never loads (a model that silently lacks its QKV biases
runs and writes fluent nonsense: loader.py:105-114).

Matrices are kept in the compute dtype (bfloat16, or float32 for the 32-bit
path), vectors (norm weights, biases) in float32, integer tables in int32.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterator, List, Tuple

import torch

from ..parts import ModelPlan, Part, WeightSpec


class WeightsError(ValueError):
    """A checkpoint that does not fit the model; lists every fault found."""

    def __init__(self, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, tuple, tuple]], where: str) -> None:
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"the weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  {len(self.missing)} missing: " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  {len(self.unexpected)} unexpected (no slot in this architecture): "
                         + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  {len(self.wrong_shape)} of a wrong shape: " + ", ".join(
                f"{n} is {tuple(got)}, expected {tuple(exp)}" for n, got, exp in self.wrong_shape))
        super().__init__("\n".join(lines))


def expected_tensors(plan: ModelPlan) -> Dict[str, Tuple[Part, str, WeightSpec]]:
    """checkpoint name -> (part, the part's local name, spec)."""
    out: Dict[str, Tuple[Part, str, WeightSpec]] = {}
    for prefix, part in plan.named_parts():
        for local, spec in part.weight_specs().items():
            out[prefix + local] = (part, local, spec)
    return out


def shard_files(model_dir: Path) -> Iterator[Path]:
    """Index file if present, else ``model.safetensors``, else ``model-*.safetensors``
    (python/helios/exec/loader.py:43-61)."""
    index = model_dir / "model.safetensors.index.json"
    if index.exists():
        with open(index, "r", encoding="utf-8") as f:
            mapping = json.load(f)["weight_map"]
        for name in sorted(set(mapping.values())):
            yield model_dir / name
        return
    single = model_dir / "model.safetensors"
    if single.exists():
        yield single
        return
    shards = sorted(model_dir.glob("model-*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no safetensors weights found in {model_dir}")
    yield from shards


def target_dtype(spec: WeightSpec, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.kind == "matrix":
        return compute_dtype
    if spec.kind == "vector":
        return torch.float32
    if spec.kind == "table":
        return torch.int32
    raise ValueError(f"unknown weight kind {spec.kind!r}")


def bind_tensors(plan: ModelPlan, tensors: Dict[str, torch.Tensor]) -> None:
    """Hand every part its tensors (already on the device, in their final dtype)."""
    expected = expected_tensors(plan)
    per_part: Dict[int, Tuple[Part, Dict[str, torch.Tensor]]] = {}
    for name, (part, local, _spec) in expected.items():
        source = name if name in tensors else plan.tied.get(name)
        per_part.setdefault(id(part), (part, {}))[1][local] = tensors[source]
    for part, local_tensors in per_part.values():
        part.bind(local_tensors)


def load_weights(plan: ModelPlan, model_dir, compute_dtype: torch.dtype, device) -> None:
    """Read the checkpoint of ``model_dir`` into the parts of ``plan``."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    expected = expected_tensors(plan)
    tensors: Dict[str, torch.Tensor] = {}
    unexpected: List[str] = []
    wrong: List[Tuple[str, tuple, tuple]] = []
    for shard in shard_files(model_dir):
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for key in f.keys():
                if key not in expected:
                    if not any(key.endswith(s) for s in plan.benign_suffixes):
                        unexpected.append(key)
                    continue
                spec = expected[key][2]
                shape = tuple(f.get_slice(key).get_shape())
                if shape != tuple(spec.shape):
                    wrong.append((key, shape, tuple(spec.shape)))
                    continue
                t = f.get_tensor(key)
                # copy as stored, convert on the device (a cast on the host runs at a fraction of the copy's rate)
                tensors[key] = t.to(device=device).to(dtype=target_dtype(spec, compute_dtype))
    wrong_names = {n for n, _, _ in wrong}
    missing = [n for n in expected
               if n not in tensors and n not in wrong_names
               and not (n in plan.tied and plan.tied[n] in tensors)]
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, wrong, str(model_dir))
    bind_tensors(plan, tensors)
