"""One registry from an architecture's name (``architectures[0]`` of
``config.json``) to its configuration class and its model builder.

The reference has no registry: it builds the same model for every config and
looks at ``architectures`` only to infer the QKV bias
(python/helios/exec/model.py:88-92).  Here an unknown name is an error that lists
the known ones, and a test can register an architecture of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]   # config.json dict -> typed config
    build_plan: Callable[[Any], Any]                # typed config -> parts.ModelPlan
    # sizes asked for on the command line (``make-toy-model``: vocab_size, hidden_size,
    # intermediate_size, layers, heads, kv_heads, head_dim, max_pos, rope_theta, rope_scaling,
    # rms_eps, sliding_window, max_window_layers, tie; None where not given) -> config.json
    toy_config: Optional[Callable[[Dict[str, Any]], Dict[str, Any]]] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_plan, *, toy_config=None,
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_plan, toy_config)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def _builtin() -> None:
    """The architectures this package ships register themselves on import."""
    from .. import models  # noqa: F401


def known_architectures():
    _builtin()
    return sorted(_ARCHITECTURES)


def find_architecture(name: str) -> Architecture:
    """By its registered name, or by a shorter name that only one registered name begins
    with, whatever the case (``llama`` finds ``LlamaForCausalLM``)."""
    _builtin()
    if name in _ARCHITECTURES:
        return _ARCHITECTURES[name]
    hits = [a for n, a in sorted(_ARCHITECTURES.items()) if n.lower().startswith(name.lower())]
    if len(hits) == 1:
        return hits[0]
    raise ConfigError(f"architecture {name!r} " + ("is ambiguous" if hits else "is not supported")
                      + "; known: " + ", ".join(known_architectures()))


def resolve_architecture(cfg: Dict[str, Any]) -> Architecture:
    _builtin()
    archs = cfg.get("architectures") or []
    if not archs:
        raise ConfigError("config.json lacks 'architectures'; known: "
                          + ", ".join(known_architectures()))
    for name in archs:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise ConfigError(f"architecture {archs[0]!r} is not supported; known: "
                      + ", ".join(known_architectures()))


def load_config(model_dir):
    """Typed configuration of the model folder, chosen by its ``architectures``."""
    cfg = read_config_json(model_dir)
    arch = resolve_architecture(cfg)
    return arch.parse_config(cfg)
