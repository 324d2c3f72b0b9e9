"""The Python entry point: ``LLMEngine`` with ``add_request / step /
run_until_complete / generate`` (python/helios/engine.py:120-470) and the shorter
``LLM(model_dir).generate(...)``."""
from __future__ import annotations

import random
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config.engine_config import EngineConfig
from ..sampling import Sampler
from .batch import StepEntry
from .core import EngineCore
from .model import DecoderModel
from .scheduler import Scheduler, SchedulerConfig, StepPlan
from .tokenizer import load_tokenizer
from .types import CompletionOutput, FinishReason, Request, SamplingParams, Sequence as Seq


class ModelExecutor:
    """Runs a scheduler's plan as ONE batch through ``EngineCore.step`` and samples
    (python/helios/exec/runner.py:108-153 runs prompts and decodes as two passes)."""

    def __init__(self, core: EngineCore) -> None:
        self.core = core
        self.sampler = Sampler()
        self.launch_steps = 0

    def run(self, plan: StepPlan) -> Dict[int, int]:
        entries = [StepEntry(i.seq_id, i.token_ids, [i.num_tokens - 1] if i.sample else [])
                   for i in plan.items]
        logits = self.core.step(entries, manage_cache=False)
        sampled = [i for i in plan.items if i.sample]
        if not sampled:
            return {}
        tokens = self.sampler.sample(logits, [i.params for i in sampled],
                                     [i.rng_seed for i in sampled],
                                     [i.rng_offset for i in sampled])
        return {i.seq_id: t for i, t in zip(sampled, tokens)}


class LLMEngine:
    def __init__(self, config: EngineConfig, model: Optional[DecoderModel] = None) -> None:
        config.validate()
        self.config = config
        self.model = model or DecoderModel.from_folder(config.model_dir, dtype=config.dtype,
                                                       device=config.device)
        mcfg = self.model.config
        num_pages = config.num_blocks or EngineCore.pages_for_bytes(
            self.model, config.block_size, config.kv_cache_bytes)
        max_len = config.max_model_len or getattr(mcfg, "max_position_embeddings", None) \
            or num_pages * config.block_size
        # a context longer than the pool is a promise that cannot be kept
        # (python/helios/engine.py:157-160)
        max_len = min(max_len, num_pages * config.block_size)
        self.max_model_len = max_len
        self.num_blocks = num_pages
        self.core = EngineCore(self.model, config.block_size, num_pages, config.max_num_seqs,
                               watermark=config.watermark, max_model_len=max_len,
                               use_cuda_graphs=config.use_cuda_graphs)
        self.scheduler = Scheduler(
            SchedulerConfig(max_num_seqs=config.max_num_seqs,
                            max_num_batched_tokens=config.max_num_batched_tokens,
                            max_model_len=max_len,
                            enable_chunked_prefill=config.enable_chunked_prefill),
            self.core.cache)
        self.executor = ModelExecutor(self.core)
        self._rng = random.Random(config.seed)
        self._tokenizer = None
        self._tokenizer_loaded = False
        self._seq_of_request: Dict[str, int] = {}
        self._completed: List[CompletionOutput] = []

    # ------------------------------------------------------------------ tokenizer
    @property
    def tokenizer(self):
        if not self._tokenizer_loaded:
            self._tokenizer = load_tokenizer(self.config.tokenizer_dir or self.config.model_dir)
            self._tokenizer_loaded = True
        if self._tokenizer is None:
            raise ValueError("the model folder has no tokenizer; pass token ids instead of text")
        return self._tokenizer

    @property
    def eos_token_ids(self) -> List[int]:
        ids = list(getattr(self.model.config, "eos_token_ids", ()) or ())
        if not ids:
            try:
                eos = self.tokenizer.eos_token_id
                ids = [eos] if eos is not None else []
            except ValueError:
                ids = []
        return [i for i in ids if 0 <= i < self.core.vocab_size]

    # ------------------------------------------------------------------ submit
    def add_request(self, request_id: str, prompt_token_ids: Sequence[int],
                    params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        for t in prompt_token_ids:
            if not 0 <= int(t) < self.core.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary")
        seed = params.seed if params.seed is not None else self._rng.getrandbits(63)
        seq_id = self.scheduler.add_request(
            Request(request_id, [int(t) for t in prompt_token_ids], params), rng_seed=seed)
        self._seq_of_request[request_id] = seq_id
        return seq_id

    def add_prompt(self, request_id: str, prompt: str, params: Optional[SamplingParams] = None) -> int:
        return self.add_request(request_id, self.tokenizer.encode(prompt), params)

    def abort(self, request_id: str) -> bool:
        seq_id = self._seq_of_request.get(request_id)
        return False if seq_id is None else self.scheduler.abort(seq_id)

    # ------------------------------------------------------------------ run
    def step(self) -> List[CompletionOutput]:
        """One scheduler iteration; returns the requests that completed in it."""
        self.scheduler.step(self.executor)
        self._apply_stop_strings()
        done = [self._make_output(seq) for seq in self.scheduler.take_finished()]
        self._completed.extend(done)
        return done

    def run_until_complete(self, max_steps: int = 100_000) -> List[CompletionOutput]:
        results: List[CompletionOutput] = []
        steps = 0
        while self.scheduler.has_work and steps < max_steps:
            results.extend(self.step())
            steps += 1
        return results

    def generate(self, prompts: Union[Sequence[str], Sequence[Sequence[int]]],
                 params: Union[None, SamplingParams, Sequence[SamplingParams]] = None
                 ) -> List[CompletionOutput]:
        """Submit all prompts (texts or lists of token ids), run to completion, return the
        results in the order of the prompts (python/helios/engine.py:459-470)."""
        order = {}
        for i, prompt in enumerate(prompts):
            p = params[i] if isinstance(params, (list, tuple)) else params
            rid = f"batch-{i}"
            order[rid] = i
            if isinstance(prompt, str):
                self.add_prompt(rid, prompt, p)
            else:
                self.add_request(rid, prompt, p)
        results = self.run_until_complete()
        return sorted((r for r in results if r.request_id in order),
                      key=lambda r: order[r.request_id])

    # ------------------------------------------------------------------ helpers
    def _apply_stop_strings(self) -> None:
        """Finish a request whose text now holds one of its stop strings, cut before it
        (python/helios/engine.py:395-423)."""
        for seq in list(self.scheduler.running):
            stops = seq.request.params.stop
            if not stops or not seq.output_token_ids:
                continue
            try:
                text = self.tokenizer.decode(seq.output_token_ids)
            except ValueError:
                return
            cut = min((text.find(s) for s in stops if s and s in text), default=-1)
            if cut >= 0:
                seq.output_text_override = text[:cut]
                self.scheduler._finish(seq, FinishReason.STOP)

    def _make_output(self, seq: Seq) -> CompletionOutput:
        if seq.output_text_override is not None:
            text = seq.output_text_override
        else:
            try:
                text = self.tokenizer.decode(seq.output_token_ids) if seq.output_token_ids else ""
            except Exception:
                text = ""
        return CompletionOutput(seq.request.request_id, list(seq.output_token_ids), text,
                                seq.finish_reason, seq.prompt_len)

    def stats_snapshot(self) -> Dict[str, float]:
        s = self.scheduler.stats
        pools = self.core.cache.pools
        return {
            "helios_steps": s.steps, "helios_prefill_tokens": s.prefill_tokens,
            "helios_decode_tokens": s.decode_tokens, "helios_preemptions": s.preemptions,
            "helios_finished": s.finished, "helios_running": len(self.scheduler.running),
            "helios_waiting": len(self.scheduler.waiting),
            "helios_pages_used": sum(p.num_used for p in pools),
            "helios_pages_total": sum(p.num_pages for p in pools),
        }


class LLM:
    """``LLM(model_dir, dtype=..., kv_cache_bytes=...).generate(prompts, SamplingParams(...))``."""

    def __init__(self, model_dir: str, **engine_options) -> None:
        self.engine = LLMEngine(EngineConfig(model_dir=str(model_dir), **engine_options))

    def generate(self, prompts=None, sampling_params=None, prompt_token_ids=None):
        if (prompts is None) == (prompt_token_ids is None):
            raise ValueError("give either prompts or prompt_token_ids")
        return self.engine.generate(prompts if prompts is not None else prompt_token_ids,
                                    sampling_params)
