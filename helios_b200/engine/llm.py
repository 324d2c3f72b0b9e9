"""The Python entry point: ``LLMEngine`` with ``add_request / step /
run_until_complete / generate`` (python/helios/engine.py:120-470) and the shorter
``LLM(model_dir).generate(...)``."""
from __future__ import annotations

import random
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config.engine_config import EngineConfig
from ..sampling import Sampler
from .batch import StepEntry
from .core import EngineCore
from .model import DecoderModel
from .scheduler import ExecFault, Scheduler, SchedulerConfig, StepPlan
from .tokenizer import load_tokenizer
from .types import CompletionOutput, FinishReason, Request, SamplingParams, Sequence as Seq


class _TokenMailbox:
    """Pinned host memory that a step's sampled tokens are copied into, and the event
    that says the copy is done."""

    def __init__(self, capacity: int) -> None:
        self.host = torch.empty(capacity, dtype=torch.int32, pin_memory=True)
        self.event = torch.cuda.Event()
        self.busy = False


class StepHandle:
    """A step that has been enqueued on the device.  ``device_tokens`` (int32, one per
    sampled item, in the plan's order) can feed the next step at once; ``result()`` waits
    for this step alone and gives seq_id -> token."""

    def __init__(self, seq_ids: List[int], device_tokens: Optional[torch.Tensor],
                 mailbox: Optional[_TokenMailbox]) -> None:
        self.seq_ids = seq_ids
        self.device_tokens = device_tokens
        self._mailbox = mailbox

    def result(self) -> Dict[int, int]:
        if self._mailbox is None:
            return {}
        self._mailbox.event.synchronize()
        tokens = self._mailbox.host[:len(self.seq_ids)].tolist()
        self._mailbox.busy = False
        return dict(zip(self.seq_ids, tokens))

    def discard(self) -> None:
        """Nobody will read the tokens; the mailbox may be used again once its copy is done."""
        if self._mailbox is not None:
            self._mailbox.busy = False


class ModelExecutor:
    """Runs a scheduler's plan as ONE batch through ``EngineCore.step`` and samples
    (python/helios/exec/runner.py:108-153 runs prompts and decodes as two passes).
    ``launch`` only enqueues the work: the host is free to prepare the next step while
    the device runs this one."""

    def __init__(self, core: EngineCore, max_num_seqs: int = 64) -> None:
        self.core = core
        self.sampler = Sampler()
        self._capacity = max(1, max_num_seqs)
        self._mailboxes: List[_TokenMailbox] = []

    def _mailbox(self) -> _TokenMailbox:
        for m in self._mailboxes:
            if not m.busy:
                break
        else:
            m = _TokenMailbox(self._capacity)
            self._mailboxes.append(m)
        m.event.synchronize()         # a copy whose result nobody fetched
        m.busy = True
        return m

    def launch(self, plan: StepPlan, feed: Optional[StepHandle] = None) -> StepHandle:
        """``feed``: the handle of the step before, when the plan's tokens are the ones that
        step samples (``PlanItem.fed_on_device``): they are taken on the device."""
        entries = [StepEntry(i.seq_id, i.token_ids, [i.num_tokens - 1] if i.sample else [])
                   for i in plan.items]
        on_device = [i.fed_on_device for i in plan.items]
        token_feed = None
        if any(on_device):
            if not all(on_device) or feed is None or feed.seq_ids != [i.seq_id for i in plan.items]:
                raise ValueError("a step fed on the device needs the handle of the step that "
                                 "samples exactly its requests, in its order")
            token_feed = feed.device_tokens
        logits = self.core.step(entries, manage_cache=False, token_feed=token_feed)
        sampled = [i for i in plan.items if i.sample]
        if not sampled:
            return StepHandle([], None, None)
        if len(sampled) > self._capacity:
            self._capacity = len(sampled)
            self._mailboxes = [m for m in self._mailboxes if m.busy]
        tokens = self.sampler.sample_device(logits, [i.params for i in sampled],
                                            [i.rng_seed for i in sampled],
                                            [i.rng_offset for i in sampled])
        box = self._mailbox()
        if box.host.numel() < len(sampled):
            box.host = torch.empty(self._capacity, dtype=torch.int32, pin_memory=True)
        box.host[:len(sampled)].copy_(tokens, non_blocking=True)
        box.event.record()
        return StepHandle([i.seq_id for i in sampled], tokens, box)

    def run(self, plan: StepPlan) -> Dict[int, int]:
        return self.launch(plan).result()


class LLMEngine:
    def __init__(self, config: EngineConfig, model: Optional[DecoderModel] = None) -> None:
        config.validate()
        self.config = config
        self.model = model or DecoderModel.from_folder(config.model_dir, dtype=config.dtype,
                                                       device=config.device)
        mcfg = self.model.config
        from ..cache.manager import cache_groups_of
        specs, _ = cache_groups_of(self.model.plan)
        if config.num_blocks:
            num_pages = [config.num_blocks] * len(specs)
        else:
            num_pages = EngineCore.pages_for_bytes(
                self.model, config.block_size, config.kv_cache_bytes, config.max_num_seqs,
                config.max_num_batched_tokens)
        # a context longer than the pool is a promise that cannot be kept
        # (python/helios/engine.py:157-160); only the groups that keep every key bound it:
        # where every layer has a window, the window buys any length
        keeps_all = [n for n, s in zip(num_pages, specs) if s.window is None]
        pool_tokens = min(keeps_all) * config.block_size if keeps_all else None
        max_len = config.max_model_len or getattr(mcfg, "max_position_embeddings", None) \
            or pool_tokens or max(num_pages, default=8) * config.block_size
        if pool_tokens is not None:
            max_len = min(max_len, pool_tokens)
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
        self.executor = ModelExecutor(self.core, config.max_num_seqs)
        # a decode step that is launched while the one before still runs: (plan, handle)
        self._in_flight = None
        self.steps_ahead = 0
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
        """One scheduler iteration; returns the requests that completed in it.

        With ``run_ahead`` the next decode step is enqueued before this one's tokens are
        read: its token ids are taken from this step's samples on the device, so the device
        does not wait while the host reads tokens and prepares the next batch.  A request
        that stops on the token being read has one more token computed in vain."""
        sched = self.scheduler
        if self._in_flight is None:
            plan = sched.schedule()
            if plan.is_empty:
                return self._collect()
            try:
                handle = self.executor.launch(plan)
            except ExecFault as fault:
                sched.fault(plan, fault)
                return self._collect()
            sched.launched(plan)
        else:
            plan, handle = self._in_flight
            self._in_flight = None
        ahead = ahead_handle = None
        if self.config.run_ahead:
            ahead = sched.schedule_ahead(plan)
            if ahead is not None:
                try:
                    ahead_handle = self.executor.launch(ahead, feed=handle)
                except ExecFault as fault:
                    sched.fault(ahead, fault)
                    ahead = None
                else:
                    sched.launched(ahead)
                    self.steps_ahead += 1
        sched.complete(plan, handle.result(), ahead)
        self._apply_stop_strings()
        if ahead is not None:
            if any(not sched.seqs[i.seq_id].is_finished for i in ahead.items):
                self._in_flight = (ahead, ahead_handle)
            else:
                ahead_handle.discard()
        return self._collect()

    def _collect(self) -> List[CompletionOutput]:
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
