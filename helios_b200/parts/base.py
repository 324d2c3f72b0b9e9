"""Interfaces of the parts a model is put together from.

A model is a list of blocks; a block arranges a mixer and a feed-forward between
norms; a position encoding serves whichever part asks for it.  Every part takes
its sizes and constants as constructor parameters and does not know which model
it is in: the plan builder of an architecture (``helios_b200/models``) reads the
typed configuration and hands each part its numbers, layer by layer.

What a part must provide
------------------------
``weight_specs()``  local tensor name -> ``WeightSpec`` (shape, kind, init).  The
                    loader joins the part's prefix in the plan with the local
                    name to get the checkpoint name.
``bind(tensors)``   receives its tensors on the device in their final dtype
                    (matrices in the compute dtype, vectors in float32, integer
                    tables in int32) and may fuse or re-lay them.
``forward(...)``    see each base class.

A mixer also says what it keeps between steps: ``cache_spec()`` (keys and values
per token, in pages, all of them or a window) and ``state_spec()`` (a tensor of
fixed size per request, in a slot).  The cache manager sizes pools and slots
from these alone.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class WeightSpec:
    shape: Tuple[int, ...]
    kind: str = "matrix"      # "matrix": compute dtype | "vector": float32 | "table": int32
    init: str = "normal"      # "normal": N(0, std) | "ones_jitter": 1 + N(0, std) | "ones" | "zeros"
    std: float = 0.02


@dataclass(frozen=True)
class PagedCacheSpec:
    """Keys and values a mixer stores for every token."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every key is needed; W: only the last W


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size a mixer keeps per request."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """The pages of one cache id, as a mixer sees them."""
    k_pages: torch.Tensor         # [pages, kv heads, page_size, head_dim]
    v_pages: torch.Tensor
    group: int                    # index into StepContext.block_tables
    page_size: int
    write: bool = True            # False: this run reads what another run wrote


class Part:
    #: False for a part whose forward depends on host values of the batch; a step
    #: with such a part is never captured into a CUDA graph.
    graph_safe = True

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors")

    def kernel_libraries(self, dtype: torch.dtype) -> Iterable[str]:
        """Names of the kernel libraries (``csrc.build.LIBRARIES``) this part's ops run on
        at its sizes, so that a model compiles them together when it is made; a library
        that is not named is compiled when an op first asks for it."""
        return ()


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                    out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += delta`` in float32 (in place, unless ``rows`` selects) and the
        normed rows in ``out_dtype``.  The default does it in two steps."""
        if rows is not None:
            r = residual.index_select(0, rows.long())
            if delta is not None:
                r = r + delta.index_select(0, rows.long()).float()
            return self.forward(r.to(out_dtype))
        if delta is not None:
            residual.add_(delta.float())
        return self.forward(residual.to(out_dtype))


class PositionEncoding(Part):
    def prepare(self, ctx) -> None:
        """Called once per step before the layers for the plan's own encoding; may leave
        tables on ``ctx`` for the mixers that were given no encoding of their own."""

    def tables(self, ctx):
        """What a mixer that was handed THIS encoding reads for the step's tokens, made at
        most once per step and kept in ``ctx.step_tables`` under the encoding's identity: so
        a model may hold several encodings (another base on every other layer) and each mixer
        gets its own.  Default: nothing."""
        return None

    def embed(self, ctx, hidden: torch.Tensor) -> torch.Tensor:
        """An additive encoding changes the embedded tokens here; default: nothing."""
        return hidden


class InputStage(Part):
    """Turns the step's token ids into the float32 residual stream [T, width].  The plain
    one is a table look-up (``TokenEmbedding``); a scale or anything else an architecture
    does before its first block is a subclass."""

    #: ids must lie in [0, vocab_size)
    vocab_size: int = 0

    def forward(self, ctx) -> torch.Tensor:
        raise NotImplementedError


class OutputStage(Part):
    """Turns the residual stream into float32 logits [wanted, vocab] at ``ctx.want_rows``
    only.  The plain one (``NormedHead``) is a final norm and a projection; a missing norm,
    a cap on the logits or a bias is a subclass.  It may be made of several parts with
    tensors: ``named_parts`` gives (checkpoint prefix, part) for each."""

    def named_parts(self) -> List[Tuple[str, Part]]:
        return []

    def forward(self, ctx, residual: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError


@dataclass
class DeferredNorm:
    """An RMS norm of the residual stream that the part BEFORE the norm has all but done
    while it added its output: the rows times the norm weight, and partial sums of their
    squares, from which the part AFTER the norm takes each row's 1 / rms as a factor on its
    first product.  Handed from one ``forward_from_residual`` to the next."""
    norm: "Norm"                  # the norm it stands for (its weight and eps went in)
    scaled: torch.Tensor          # compute dtype [T, width]: residual * norm weight
    sumsq: torch.Tensor           # float32 [T, slots]: they add up to sum(residual ** 2) per row


class Mixer(Part):
    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, ctx, x: torch.Tensor, cache: Optional[LayerCache],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        """x: [T, width] in the compute dtype, the batch described by ``ctx``
        (``engine.batch.StepContext``); returns [T, width].  ``state`` is
        [slots, *state_spec.shape]; a request's row is ``ctx.slots[seq]``."""
        raise NotImplementedError

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm: "Norm",
                              cache: Optional[LayerCache], state: Optional[torch.Tensor],
                              pre: Optional[DeferredNorm] = None, then: Optional["Norm"] = None):
        """Optional fusion with the norm before and the add after: apply ``norm`` to the
        float32 residual stream (to which nothing is pending), run, and ADD the output to
        ``residual`` in place.  Return False, having done nothing, where the part has no such
        path for this step; the block then norms, calls ``forward`` and adds as usual.

        ``pre``: ``norm`` of this very residual, all but done by the part before (it may be
        ignored).  ``then``: the norm that will be applied to the residual next, if the block
        knows it; a part that can may return a ``DeferredNorm`` for it instead of True."""
        return False


class FeedForward(Part):
    def state_spec(self) -> Optional[StateSpec]:
        """A feed-forward may keep a tensor of fixed size per request too; it then finds it
        in ``ctx.part_state(self)`` as [slots, *shape]."""
        return None

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm: "Norm",
                              pre: Optional[DeferredNorm] = None, then: Optional["Norm"] = None):
        """As ``Mixer.forward_from_residual``: norm, run and add in place (True, or a
        ``DeferredNorm`` for ``then``), or return False."""
        return False


class Block:
    """Arrangement of parts in one layer."""

    def named_parts(self) -> List[Tuple[str, Part]]:
        """(prefix below the layer's own prefix, part) for every part with tensors."""
        raise NotImplementedError

    @property
    def mixer(self) -> Optional[Mixer]:
        return None

    @property
    def first_norm(self) -> Optional["Norm"]:
        """The norm this block applies to the residual stream before anything else, if it
        starts that way and accepts a ``DeferredNorm`` for it in place of ``delta``; the
        model tells the block before (``ctx.norm_after_block``)."""
        return None

    def state_specs(self) -> List[Tuple[Part, StateSpec]]:
        """(part, spec) of every part of the block OTHER than the mixer that keeps a tensor of
        fixed size per request slot (the mixer's comes to ``forward`` as ``state``).  The cache
        manager makes one tensor [slots, *shape] per schedule entry and part, zeroed when a slot
        is handed out; the part finds it in ``ctx.part_state(part)`` while its block runs."""
        out = []
        for _prefix, part in self.named_parts():
            spec = getattr(part, "state_spec", lambda: None)()
            if spec is not None and part is not self.mixer:
                out.append((part, spec))
        return out

    def forward(self, ctx, residual: torch.Tensor, delta: Optional[torch.Tensor],
                cache: Optional[LayerCache], state: Optional[torch.Tensor]):
        """Takes the float32 residual stream and the not-yet-added output of the
        block before (or None; or, for a block with ``first_norm``, a ``DeferredNorm`` of
        it); returns the pair for the next block."""
        raise NotImplementedError


# ---------------------------------------------------------------------- registries
_PART_KINDS: Dict[str, Dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "block": {},
}


def register_part(kind: str, name: str, cls: type, *, replace: bool = False) -> None:
    table = _PART_KINDS[kind]
    if name in table and not replace:
        raise ValueError(f"{kind} {name!r} is already registered")
    table[name] = cls


def part_class(kind: str, name: str) -> type:
    try:
        return _PART_KINDS[kind][name]
    except KeyError:
        known = ", ".join(sorted(_PART_KINDS.get(kind, {}))) or "none"
        raise ValueError(f"no {kind} named {name!r}; known: {known}") from None


def known_parts(kind: str) -> List[str]:
    return sorted(_PART_KINDS[kind])
