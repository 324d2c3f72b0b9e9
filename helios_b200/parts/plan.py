"""The plan of a model: its parts, their checkpoint prefixes, and the order in
which the layers run.

The order is data: ``schedule`` is a list of ``Run`` entries.  An entry names a
layer (the same layer may be named twice: its weights then run twice) and a
cache id.  By default every entry has a cache of its own; an entry may instead
name the cache id of an earlier entry and read what that run wrote
(``writes_cache=False``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Tuple

from .base import Block, Norm, Part, PositionEncoding
from .embedding import OutputHead, TokenEmbedding


@dataclass(frozen=True)
class Run:
    layer: int
    cache: Optional[int] = None        # None: this entry's own index in the schedule
    writes_cache: bool = True


@dataclass
class ModelPlan:
    config: Any
    embedding: TokenEmbedding
    position: Optional[PositionEncoding]
    layers: List[Block]
    layer_prefixes: List[str]
    final_norm: Norm
    head: OutputHead
    schedule: List[Run] = field(default_factory=list)
    embedding_prefix: str = "model.embed_tokens."
    position_prefix: str = "model.position."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."
    # checkpoint name -> name whose tensor stands in when the first is absent
    tied: Dict[str, str] = field(default_factory=dict)
    # suffixes of checkpoint tensors that are buffers, not weights
    benign_suffixes: Tuple[str, ...] = (".rotary_emb.inv_freq", ".attn.bias", ".attn.masked_bias")

    def __post_init__(self) -> None:
        if not self.schedule:
            self.schedule = [Run(i) for i in range(len(self.layers))]
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {run.layer} of {len(self.layers)}")
            cid = self.cache_id(i)
            if cid != i:
                if not 0 <= cid < i:
                    raise ValueError(f"schedule entry {i} reads cache {cid}, which no earlier entry owns")
                if run.writes_cache:
                    raise ValueError(f"schedule entry {i} shares cache {cid} and must not write it")

    def cache_id(self, entry: int) -> int:
        run = self.schedule[entry]
        return entry if run.cache is None else run.cache

    def named_parts(self) -> Iterator[Tuple[str, Part]]:
        """(checkpoint prefix, part) of every part that may own tensors."""
        yield self.embedding_prefix, self.embedding
        if self.position is not None:
            yield self.position_prefix, self.position     # tensors only if the encoding is learned
        for prefix, block in zip(self.layer_prefixes, self.layers):
            for sub, part in block.named_parts():
                yield prefix + sub, part
        yield self.final_norm_prefix, self.final_norm
        yield self.head_prefix, self.head

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for _, part in self.named_parts())
