"""Engine options (python/helios/engine.py:33-62, without the options of parts
this package does not have: prefix cache, speculation, quantised formats)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineConfig:
    model_dir: str
    kv_cache_bytes: int = 512 * 1024 * 1024
    block_size: int = 16
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    max_model_len: Optional[int] = None      # None -> max_position_embeddings
    device: str = "cuda:0"
    dtype: str = "bfloat16"                  # "bfloat16" | "float32"
    enable_chunked_prefill: bool = True
    watermark: float = 0.01
    tokenizer_dir: Optional[str] = None
    num_blocks: Optional[int] = None         # overrides kv_cache_bytes when given
    seed: int = 0                            # seeds requests that bring no seed
    use_cuda_graphs: bool = True
    run_ahead: bool = True                   # enqueue the next decode step before reading this one's tokens

    def validate(self) -> None:
        if self.block_size <= 0:
            raise ValueError("block_size must be positive")
        if self.max_num_seqs <= 0:
            raise ValueError("max_num_seqs must be positive")
        if self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if not 0.0 <= self.watermark < 1.0:
            raise ValueError("watermark must be in [0, 1)")
