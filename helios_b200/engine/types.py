"""Requests, sequences and results (python/helios/core/types.py:41-211)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional


class SeqState(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"
    ABORTED = "aborted"


class FinishReason(Enum):
    STOP = "stop"          # a stop token id (kept in the output)
    LENGTH = "length"      # max_tokens, max_model_len, or the cache is too small to go on
    ABORTED = "aborted"


@dataclass
class SamplingParams:
    """How a request's tokens are chosen and when it stops.  Names, defaults and limits are
    the reference's (python/helios/core/types.py:58-85), so that its callers need no change."""

    max_tokens: int = 128
    temperature: float = 0.0      # 0 = greedy
    top_p: float = 1.0
    top_k: int = 0                # 0 disables
    stop: List[str] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    seed: Optional[int] = None

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    def validate(self) -> None:
        limits = (
            (self.max_tokens > 0, "max_tokens must be positive"),
            (self.temperature >= 0.0, "temperature must be >= 0"),
            (0.0 < self.top_p <= 1.0, "top_p must be in (0, 1]"),
            (self.top_k >= 0, "top_k must be >= 0"),
        )
        for ok, message in limits:
            if not ok:
                raise ValueError(message)


@dataclass
class Request:
    request_id: str
    prompt_token_ids: List[int]
    params: SamplingParams
    arrival_step: int = 0

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_token_ids)


@dataclass(eq=False)       # an entity: two sequences are equal only if they are the same object
class Sequence:
    """Scheduler-side state of one request (python/helios/core/types.py:105-195)."""

    seq_id: int
    request: Request
    state: SeqState = SeqState.WAITING
    output_token_ids: List[int] = field(default_factory=list)
    num_computed_tokens: int = 0          # tokens whose keys and values are in the cache
    finish_reason: Optional[FinishReason] = None
    first_token_step: Optional[int] = None
    last_token_step: Optional[int] = None
    preempt_count: int = 0
    rng_seed: int = 0                     # the request's seed, or one the engine drew
    output_text_override: Optional[str] = None

    @property
    def prompt_len(self) -> int:
        return self.request.prompt_len

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def total_tokens(self) -> int:
        return self.prompt_len + len(self.output_token_ids)

    @property
    def num_pending_tokens(self) -> int:
        """Tokens still to be run: the whole prompt at first, one token while decoding,
        prompt and outputs again after a preemption."""
        return self.total_tokens - self.num_computed_tokens

    @property
    def is_finished(self) -> bool:
        return self.state in (SeqState.FINISHED, SeqState.ABORTED)

    def all_token_ids(self) -> List[int]:
        return self.request.prompt_token_ids + self.output_token_ids

    def token_slice(self, start: int, n: int) -> List[int]:
        """``all_token_ids()[start:start + n]`` without building the whole list (a decoding
        request with a long prompt would copy it every step)."""
        prompt, outputs = self.request.prompt_token_ids, self.output_token_ids
        split = len(prompt)
        if start + n <= split:
            return prompt[start:start + n]
        if start >= split:
            return outputs[start - split:start - split + n]
        return prompt[start:] + outputs[:start + n - split]

    def reset_for_recompute(self) -> None:
        """Its cache is gone; the outputs made so far are kept and are run again with
        the prompt (python/helios/core/types.py:181-191)."""
        self.num_computed_tokens = 0
        self.state = SeqState.PREEMPTED
        self.preempt_count += 1


@dataclass
class CompletionOutput:
    request_id: str
    token_ids: List[int]
    text: str = ""
    finish_reason: Optional[FinishReason] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0        # always 0: there is no prefix cache (python/helios/core/types.py:207)

    @property
    def completion_tokens(self) -> int:
        return len(self.token_ids)
