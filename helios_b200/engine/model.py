"""A model on the device: a plan with its tensors bound, and the forward pass of
one step (python/helios/exec/model.py:465-496 ``forward_batched``)."""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch

from .. import models as _models  # registers the architectures
from ..config.registry import resolve_architecture
from ..config.model_config import read_config_json
from ..parts import ModelPlan
from ..weights import bind_random_weights, load_weights

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return _DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not supported (bfloat16 or float32)") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("helios_b200 runs on a CUDA device only (sm_100a); there is no CPU path. "
                           f"Asked for {device}, torch.cuda.is_available() = {torch.cuda.is_available()}")
    return device


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device: torch.device) -> None:
        self.plan = plan
        self.config = plan.config
        self.dtype = dtype
        self.device = device
        from ..csrc import ops
        ops.preload(name for _prefix, part in plan.named_parts() for name in part.kernel_libraries(dtype))

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir, dtype="bfloat16", device="cuda:0") -> "DecoderModel":
        device = require_cuda(device)
        dtype = parse_dtype(dtype)
        cfg_json = read_config_json(Path(model_dir))
        arch = resolve_architecture(cfg_json)
        plan = arch.build_plan(arch.parse_config(cfg_json))
        load_weights(plan, model_dir, dtype, device)
        return cls(plan, dtype, device)

    @classmethod
    def from_config(cls, config_json: dict, seed: int, dtype="bfloat16", device="cuda:0") -> "DecoderModel":
        """Random weights drawn on the device (no file)."""
        device = require_cuda(device)
        dtype = parse_dtype(dtype)
        arch = resolve_architecture(config_json)
        plan = arch.build_plan(arch.parse_config(config_json))
        bind_random_weights(plan, seed, dtype, device)
        return cls(plan, dtype, device)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, cache) -> Optional[torch.Tensor]:
        """Run the step's tokens through every scheduled layer (writing the cache) and
        return float32 logits [wanted, vocab] (None if nothing is wanted)."""
        plan = self.plan
        ctx.step_tables = {}
        if plan.position is not None:
            plan.position.prepare(ctx)
        residual = plan.embedding.forward(ctx)
        if plan.position is not None:
            residual = plan.position.embed(ctx, residual)
        delta = None
        runs = len(plan.schedule)
        for entry, run in enumerate(plan.schedule):
            ctx.block_states = cache.part_states(entry)
            # the norm that meets the residual stream first after this block, if the next
            # block says so: a part may prepare it while it adds its own output
            ctx.norm_after_block = (plan.layers[plan.schedule[entry + 1].layer].first_norm
                                    if entry + 1 < runs else None)
            residual, delta = plan.layers[run.layer].forward(
                ctx, residual, delta, cache.layer_cache(entry), cache.layer_state(entry))
        ctx.block_states = {}
        ctx.norm_after_block = None
        if ctx.num_wanted == 0:
            return None
        return plan.output.forward(ctx, residual, delta)
