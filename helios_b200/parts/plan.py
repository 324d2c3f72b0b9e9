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

from .base import Block, InputStage, Norm, OutputStage, Part, PositionEncoding
from .embedding import NormedHead


@dataclass(frozen=True)
class Run:
    layer: int
    cache: Optional[int] = None        # None: this entry's own index in the schedule
    writes_cache: bool = True


@dataclass
class ModelPlan:
    """``embedding`` is the input stage (token ids -> residual stream); the output stage
    (residual stream -> logits at the wanted rows) is ``output``, or, when ``final_norm`` and
    ``head`` are given instead, the usual ``NormedHead`` made of the two."""
    config: Any
    embedding: InputStage
    position: Optional[PositionEncoding]
    layers: List[Block]
    layer_prefixes: List[str]
    final_norm: Optional[Norm] = None
    head: Optional[Part] = None
    schedule: List[Run] = field(default_factory=list)
    output: Optional[OutputStage] = None
    embedding_prefix: str = "model.embed_tokens."
    position_prefix: str = "model.position."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."
    # checkpoint name -> name whose tensor stands in when the first is absent
    tied: Dict[str, str] = field(default_factory=dict)
    # suffixes of checkpoint tensors that are buffers, not weights
    benign_suffixes: Tuple[str, ...] = (".rotary_emb.inv_freq", ".attn.bias", ".attn.masked_bias")

    def __post_init__(self) -> None:
        if self.output is None:
            if self.final_norm is None or self.head is None:
                raise ValueError("a plan needs an output stage, or a final norm and a head")
            self.output = NormedHead(self.final_norm, self.head, self.final_norm_prefix,
                                     self.head_prefix)
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
        yield from self.output.named_parts()

    @property
    def vocab_size(self) -> int:
        """Token ids a step may bring: the configuration's ``vocab_size``, else the input
        stage's."""
        return int(getattr(self.config, "vocab_size", 0) or self.embedding.vocab_size)

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for _, part in self.named_parts())
