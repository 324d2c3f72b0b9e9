"""Traces for replay tests: how requests are cut into steps, how a trace is run
(in this process through ``EngineCore.step``, or through ``bin/trace_run`` as a
user runs it), and how every returned row is compared with the plain model."""
from __future__ import annotations

import json
import random
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def round64(n):
    return -(-n // 64) * 64


class TraceBuilder:
    """Collects steps; remembers which (request, position) every wanted row is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[tuple]] = {}     # step -> [(request, position)]
        self.fed: Dict[str, int] = {}              # request -> tokens fed so far
        self.live_tokens_peak = 0
        self._final: Dict[str, int] = {}

    def declare(self, rid: str, total: int):
        self._final[rid] = total

    def add_step(self, parts: Sequence[tuple], end: Sequence[str] = ()):
        """parts: (request, tokens of this step, want: local indices)."""
        step = len(self.steps)
        entries, rows = [], []
        for rid, toks, want in parts:
            p0 = self.fed.get(rid, 0)
            entries.append({"id": rid, "tokens": list(toks), "want": list(want)})
            rows.extend((rid, p0 + w) for w in want)
            self.fed[rid] = p0 + len(toks)
        live = [r for r in self.fed if r not in getattr(self, "_ended", set())]
        self.live_tokens_peak = max(self.live_tokens_peak,
                                    sum(round64(self._final.get(r, self.fed[r])) for r in live))
        self.steps.append({"step": step, "entries": entries, "end": list(end)})
        if rows:
            self.rows[step] = rows
        self._ended = getattr(self, "_ended", set()) | set(end)


def whole(tb: TraceBuilder, rid, toks):
    tb.declare(rid, len(toks))
    tb.add_step([(rid, toks, range(len(toks)))], end=[rid])


def prefill_then_decode(tb: TraceBuilder, rid, toks, n_decode=32):
    tb.declare(rid, len(toks))
    n0 = max(1, len(toks) - n_decode)
    tb.add_step([(rid, toks[:n0], [n0 - 1])])
    for i in range(n0, len(toks)):
        tb.add_step([(rid, toks[i:i + 1], [0])], end=[rid] if i == len(toks) - 1 else [])
    if n0 == len(toks):
        tb.add_step([], end=[rid])


def portions(tb: TraceBuilder, rid, toks, sizes):
    """Portions of the given sizes in turn (the last one takes what is left)."""
    tb.declare(rid, len(toks))
    i, k = 0, 0
    while i < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - i)
        k += 1
        tb.add_step([(rid, toks[i:i + n], range(n))], end=[rid] if i + n == len(toks) else [])
        i += n


def mixed(tb: TraceBuilder, requests: Dict[str, List[int]], seed: int, max_live=4,
          decode_tail=12, portion_choices=(2, 3, 5, 8, 13, 21, 34)):
    """Up to ``max_live`` requests at a time: portions of the prompts of some beside single
    decoded tokens of others; a request may sit a step out; a finished request ends and
    the next one starts, so pages are used again."""
    rng = random.Random(seed)
    waiting = list(requests)
    for rid in waiting:
        tb.declare(rid, len(requests[rid]))
    live: List[str] = []
    pos = {rid: 0 for rid in requests}
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        parts, ended = [], []
        for rid in list(live):
            toks = requests[rid]
            left = len(toks) - pos[rid]
            if len(live) > 1 and rng.random() < 0.2 and parts:
                continue                      # sits this step out
            if left <= decode_tail:
                n = 1
            else:
                n = min(rng.choice(portion_choices), left - decode_tail) if left - decode_tail >= 2 else left - decode_tail
            chunk = toks[pos[rid]:pos[rid] + n]
            want = list(range(n)) if n <= 3 else sorted({0, n - 1, rng.randrange(n)})
            parts.append((rid, chunk, want))
            pos[rid] += n
            if pos[rid] == len(toks):
                ended.append(rid)
                live.remove(rid)
        if parts:
            tb.add_step(parts, end=ended)


# ---------------------------------------------------------------------- running
def run_in_process(core, tb: TraceBuilder) -> Dict[int, np.ndarray]:
    from helios_b200.engine.batch import StepEntry

    out = {}
    for st in tb.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = core.step(entries) if entries else None
        if logits is not None:
            out[st["step"]] = logits.detach().float().cpu().numpy()
        for rid in st["end"]:
            core.end(rid)
        core.cache.check_invariants()
    return out


def run_trace_run(folder, dtype, tb: TraceBuilder, out_dir, max_tokens, vocab,
                  extra_args=()) -> Dict[int, np.ndarray]:
    """Through bin/trace_run, one step at a time, waiting for every ``done``."""
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)] + list(extra_args)
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for st in tb.steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"trace_run answered {line!r} to step {st['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    out = {}
    for step in tb.rows:
        data = np.fromfile(str(Path(out_dir) / f"{step}.f32"), dtype="<f4")
        out[step] = data.reshape(-1, vocab)
    for st in tb.steps:
        if st["step"] not in tb.rows:
            assert not (Path(out_dir) / f"{st['step']}.f32").exists()
    return out


def check(tb: TraceBuilder, got: Dict[int, np.ndarray], plain: Dict[str, torch.Tensor], dtype, what):
    """plain: request -> float64 logits [len, V] of the whole sequence."""
    from conftest import assert_logits_close

    assert set(got) == set(tb.rows), f"{what}: steps with logits {sorted(got)} vs {sorted(tb.rows)}"
    for step, rows in tb.rows.items():
        want = torch.stack([plain[rid][pos] for rid, pos in rows])
        g = torch.from_numpy(np.ascontiguousarray(got[step]))
        try:
            assert_logits_close(g, want, dtype, f"{what} step {step}")
        except AssertionError as exc:
            first = _first_bad(g, want, dtype)
            raise AssertionError(f"{exc}; first wrong row of the step is (request, position) = "
                                 f"{rows[first]}; the step was {tb.steps[step]}") from None


def _first_bad(g, want, dtype):
    from conftest import BF16_RTOL, F32_ATOL

    err = (g.double() - want).abs()
    if dtype == "float32":
        bad = (err.amax(-1) > F32_ATOL)
    else:
        bad = ((err / want.abs().amax(-1, keepdim=True)).amax(-1) > BF16_RTOL)
    idx = torch.nonzero(bad)
    return int(idx[0]) if len(idx) else 0
