"""helios_b200: a single-GPU inference engine for the dense GQA decoder
(Llama 3 / Qwen2.5) on B200, after the engine of anish41338/helios."""

__version__ = "0.1.0"

_LAZY = {
    "LLM": ("helios_b200.engine.llm", "LLM"),
    "LLMEngine": ("helios_b200.engine.llm", "LLMEngine"),
    "EngineConfig": ("helios_b200.config.engine_config", "EngineConfig"),
    "SamplingParams": ("helios_b200.engine.types", "SamplingParams"),
    "CompletionOutput": ("helios_b200.engine.types", "CompletionOutput"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)
