"""Typed configuration of the dense GQA decoder, read from ``config.json``.

Every size and constant the model uses comes from here; no part of the package
holds a default for a key that ``config.json`` gives.  Keys and defaults follow
python/helios/exec/model.py:30-92 (``ModelConfig.from_hf``); ``head_dim``,
``rope_scaling`` and the sliding-window keys go beyond it.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A ``config.json`` this package cannot serve; the message names the key."""


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of type ``llama3``."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_hf(self) -> Dict[str, Any]:
        return {
            "rope_type": "llama3",
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads")


@dataclass(frozen=True)
class DenseDecoderConfig:
    """Llama 3 / Qwen2.5 hyper-parameters (python/helios/exec/model.py:30-49)."""

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    attention_bias: bool
    tie_word_embeddings: bool
    hidden_act: str
    # One entry per layer: None = the layer sees every key, W = only the last W.
    layer_windows: Tuple[Optional[int], ...]
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    max_window_layers: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    model_type: str = ""
    torch_dtype: str = "float32"

    # ------------------------------------------------------------------ derived
    @property
    def group_size(self) -> int:
        """Query heads per KV head (python/helios/exec/model.py:55-58)."""
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def attention_scale(self) -> float:
        """1/sqrt(head_dim) (python/helios/exec/model.py:166)."""
        return 1.0 / math.sqrt(self.head_dim)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_parameters(self) -> int:
        H, I, V = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = (self.q_size + 2 * self.kv_size) * H + H * self.q_size + 3 * H * I + 2 * H
        if self.attention_bias:
            per_layer += self.q_size + 2 * self.kv_size
        total = V * H + self.num_hidden_layers * per_layer + H
        if not self.tie_word_embeddings:
            total += V * H
        return total

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_hf(cls, cfg: Dict[str, Any], architecture: Optional[str] = None) -> "DenseDecoderConfig":
        for key in _REQUIRED:
            if key not in cfg:
                raise ConfigError(f"config.json lacks the required key '{key}'")
            if not isinstance(cfg[key], int) or cfg[key] <= 0:
                raise ConfigError(f"config.json key '{key}' must be a positive integer, got {cfg[key]!r}")
        archs = cfg.get("architectures") or []
        architecture = architecture or (archs[0] if archs else "")
        nh = cfg["num_attention_heads"]
        nkv = cfg.get("num_key_value_heads", nh)
        if not isinstance(nkv, int) or nkv <= 0 or nh % nkv != 0:
            raise ConfigError(
                f"'num_key_value_heads' ({nkv}) must divide 'num_attention_heads' ({nh})")
        head_dim = cfg.get("head_dim")
        if head_dim is None:
            if cfg["hidden_size"] % nh != 0:
                raise ConfigError(
                    f"'hidden_size' ({cfg['hidden_size']}) is not a multiple of "
                    f"'num_attention_heads' ({nh}) and no 'head_dim' is given")
            head_dim = cfg["hidden_size"] // nh
        if not isinstance(head_dim, int) or head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"'head_dim' must be a positive even integer, got {head_dim!r}")
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"'hidden_act' = {act!r} is not supported (only 'silu')")

        L = cfg["num_hidden_layers"]
        window = cfg.get("sliding_window")
        use_window = bool(cfg.get("use_sliding_window", False))
        max_window_layers = cfg.get("max_window_layers")
        layer_types = cfg.get("layer_types")
        if layer_types is not None:
            if len(layer_types) != L:
                raise ConfigError(f"'layer_types' has {len(layer_types)} entries for {L} layers")
            wins: List[Optional[int]] = []
            for t in layer_types:
                if t == "full_attention":
                    wins.append(None)
                elif t == "sliding_attention":
                    if not isinstance(window, int) or window <= 0:
                        raise ConfigError("'layer_types' names sliding_attention but "
                                          "'sliding_window' is not a positive integer")
                    wins.append(window)
                else:
                    raise ConfigError(f"'layer_types' entry {t!r} is not supported")
        elif use_window:
            if not isinstance(window, int) or window <= 0:
                raise ConfigError("'use_sliding_window' is true but 'sliding_window' "
                                  "is not a positive integer")
            first = L if max_window_layers is None else int(max_window_layers)
            wins = [window if i >= first else None for i in range(L)]
        else:
            wins = [None] * L
        if any(w is not None for w in wins) and architecture == "LlamaForCausalLM":
            # Llama checkpoints have no layers with a window; serving the file with one would
            # silently run another model than the one it names
            raise ConfigError("'layer_types' / 'use_sliding_window' ask for sliding-window layers, "
                              "which LlamaForCausalLM does not have (Qwen2ForCausalLM does)")

        eos = cfg.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)

        return cls(
            architecture=architecture,
            vocab_size=cfg["vocab_size"],
            hidden_size=cfg["hidden_size"],
            intermediate_size=cfg["intermediate_size"],
            num_hidden_layers=L,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
            rope_theta=float(cfg.get("rope_theta", 10000.0)),
            rope_scaling=_parse_rope_scaling(cfg.get("rope_scaling")),
            attention_bias=_infer_attention_bias(cfg),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            hidden_act=act,
            layer_windows=tuple(wins),
            sliding_window=window,
            use_sliding_window=use_window,
            max_window_layers=max_window_layers,
            bos_token_id=cfg.get("bos_token_id"),
            eos_token_ids=eos_ids,
            model_type=str(cfg.get("model_type", "")),
            torch_dtype=str(cfg.get("torch_dtype", cfg.get("dtype", "float32"))),
        )

    def to_hf(self) -> Dict[str, Any]:
        """The ``config.json`` dictionary that parses back to this configuration."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_hf() if self.rope_scaling else None,
            "attention_bias": self.attention_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            out["sliding_window"] = self.sliding_window
            out["use_sliding_window"] = self.use_sliding_window
            if self.max_window_layers is not None:
                out["max_window_layers"] = self.max_window_layers
            out["layer_types"] = ["full_attention" if w is None else "sliding_attention"
                                  for w in self.layer_windows]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                   else list(self.eos_token_ids))
        return out


def _infer_attention_bias(cfg: Dict[str, Any]) -> bool:
    """``attention_bias`` if present, else true for the qwen2 family
    (python/helios/exec/model.py:79-92)."""
    if "attention_bias" in cfg:
        return bool(cfg["attention_bias"])
    model_type = str(cfg.get("model_type", "")).lower()
    archs = " ".join(cfg.get("architectures") or []).lower()
    return model_type.startswith("qwen2") or "qwen2" in archs


def _parse_rope_scaling(rs: Optional[Dict[str, Any]]) -> Optional[RopeScaling]:
    if not rs:
        return None
    kind = rs.get("rope_type", rs.get("type"))
    if kind in (None, "default"):
        return None
    if kind != "llama3":
        raise ConfigError(f"'rope_scaling' of type {kind!r} is not supported "
                          "(supported: 'llama3', 'default')")
    try:
        return RopeScaling(
            factor=float(rs["factor"]),
            low_freq_factor=float(rs["low_freq_factor"]),
            high_freq_factor=float(rs["high_freq_factor"]),
            original_max_position_embeddings=int(rs["original_max_position_embeddings"]),
        )
    except KeyError as exc:
        raise ConfigError(f"'rope_scaling' of type 'llama3' lacks the key {exc.args[0]!r}") from None


def read_config_json(model_dir) -> Dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)
