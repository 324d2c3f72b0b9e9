"""Steps that mix prompt portions with decoded tokens run as captured CUDA graphs once their
padded shape (requests, tokens) has been seen twice.  The same steps through an engine
without graphs must give the same logits, and both must agree with the plain implementation."""
import pytest
import torch

import plain_model
from conftest import assert_logits_close, random_tokens, read_folder

pytestmark = pytest.mark.gpu


def _cores(folder, dtype, pages=120, max_len=400):
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_folder(folder, dtype=dtype)
    make = lambda graphs: EngineCore(model, page_size=8, num_pages=pages, max_slots=8, max_model_len=max_len,
                                     poison_cache=float("nan"), use_cuda_graphs=graphs)
    return make(True), make(False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_llama", "tiny_tiled", "tiny_window"])
def test_mixed_steps_as_graphs_equal_steps_kernel_by_kernel(model_folders, name, dtype):
    from helios_b200.engine.batch import StepEntry

    folder = model_folders[name]
    cfg, weights = read_folder(folder)
    with_graphs, without = _cores(folder, dtype)
    V = cfg["vocab_size"]
    seqs = {r: random_tokens(V, 160, 7 + i) for i, r in enumerate("abcd")}
    done = {r: 0 for r in seqs}
    got = {r: [] for r in seqs}          # (position, logits row) from the engine with graphs

    def step(parts):
        """parts: list of (request, tokens to feed, want the last?)"""
        entries = []
        for r, n, want in parts:
            toks = seqs[r][done[r]:done[r] + n]
            entries.append(StepEntry(r, toks, [n - 1] if want else []))
        a = with_graphs.step(entries)
        b = without.step(entries)
        wanted = [(r, done[r] + n - 1) for r, n, want in parts if want]
        if wanted:
            tol = dict(atol=1e-5, rtol=0) if dtype == "float32" else dict(atol=6e-2, rtol=6e-2)
            torch.testing.assert_close(a, b, **tol)
            for row, (r, pos) in enumerate(wanted):
                got[r].append((pos, a[row].clone()))
        else:
            assert a is None and b is None
        for r, n, _ in parts:
            done[r] += n

    # the same shapes come back again and again: 3 requests / 15 tokens (no spare token),
    # 2 requests / 20 tokens (ten spare tokens in the padding request), decode steps between
    for _ in range(6):
        step([("a", 5, True), ("b", 1, True), ("c", 9, False)])
        step([("a", 13, False), ("d", 7, True)])
        step([("a", 1, True), ("b", 1, False), ("c", 1, True), ("d", 1, True)])
    captured = [key for key, g in with_graphs._graphs.items() if g.graph is not None]
    assert any(s != t for s, t in captured), f"no mixed step was captured: {captured}"
    assert any(s == t for s, t in captured), f"no decode step was captured: {captured}"
    for r, rows in got.items():
        want = plain_model.forward_logits(cfg, weights, seqs[r][:done[r]])
        for pos, row in rows:
            assert_logits_close(row[None], want[pos:pos + 1], dtype, f"{name} request {r} position {pos}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_portions_of_a_long_prompt_run_as_graphs(model_folders, dtype):
    """Steps of 1,024 tokens (a full portion alone, or a portion beside decoded tokens that
    together fill the count) are captured too; a step that fills less than seven eighths of
    the count is not."""
    from helios_b200.engine.batch import StepEntry

    folder = model_folders["tiny_window"]
    cfg, weights = read_folder(folder)
    with_graphs, without = _cores(folder, dtype, pages=800, max_len=6200)
    with_graphs.FULL_GRAPH_EAGER_RUNS = 1        # capture at the third step of a shape, as for small steps
    V = cfg["vocab_size"]
    long = random_tokens(V, 1024 * 5 + 600, 3)
    short = {r: random_tokens(V, 40, 50 + i) for i, r in enumerate("uv")}
    for r, toks in short.items():
        for core in (with_graphs, without):
            core.step([StepEntry(r, toks[:30], [])])
    rows = []
    pos = 0
    for k in range(5):
        if k % 2 == 0:
            entries = [StepEntry("long", long[pos:pos + 1024], [1023])]
            n = 1024
        else:       # 1,022 tokens of the prompt beside two decoded tokens
            entries = [StepEntry("u", short["u"][30 + k // 2:31 + k // 2], [0]),
                       StepEntry("long", long[pos:pos + 1022], [1021]),
                       StepEntry("v", short["v"][30 + k // 2:31 + k // 2], [])]
            n = 1022
        a, b = with_graphs.step(entries), without.step(entries)
        tol = dict(atol=1e-5, rtol=0) if dtype == "float32" else dict(atol=6e-2, rtol=6e-2)
        torch.testing.assert_close(a, b, **tol)
        rows.append((pos + n - 1, a[0 if k % 2 == 0 else 1].clone()))
        pos += n
    a, b = (c.step([StepEntry("long", long[pos:pos + 600], [599])]) for c in (with_graphs, without))
    torch.testing.assert_close(a, b, **tol)
    captured = sorted(key for key, g in with_graphs._graphs.items() if g.graph is not None)
    assert (1, 1024) in captured, captured           # three full portions alone
    assert (3, 1024) in with_graphs._graphs          # 1,022 + 2 tokens of three requests, seen twice
    assert not any(t > 1024 or 512 < t < 1024 for _s, t in with_graphs._graphs), sorted(with_graphs._graphs)
    want = plain_model.forward_logits(cfg, weights, long[:pos])
    for p, row in rows:
        assert_logits_close(row[None], want[p:p + 1], dtype, f"position {p}")


def test_a_decode_token_without_a_wanted_place_keeps_the_rows_in_order(model_folders):
    from helios_b200.engine.batch import StepEntry

    folder = model_folders["tiny_llama"]
    cfg, _ = read_folder(folder)
    with_graphs, without = _cores(folder, "float32")
    toks = {r: random_tokens(cfg["vocab_size"], 40, i) for i, r in enumerate("xyz")}
    for core in (with_graphs, without):
        core.step([StepEntry(r, t[:20], []) for r, t in toks.items()])
    for k in range(20, 28):
        entries = [StepEntry("x", [toks["x"][k]], [0]), StepEntry("y", [toks["y"][k]], []),
                   StepEntry("z", [toks["z"][k]], [0])]
        a, b = with_graphs.step(entries), without.step(entries)
        assert a.shape[0] == 2
        torch.testing.assert_close(a, b, atol=1e-5, rtol=0)
    assert any(g.graph is not None for g in with_graphs._graphs.values())


@pytest.mark.parametrize("name", ["tiny_window", "tiny_tiled"])
def test_generation_with_and_without_graphs_gives_the_same_tokens(model_folders, name):
    """Requests that arrive at different steps, stop at different lengths and squeeze a
    small cache (preemptions) through the scheduler: captured steps, launching ahead, both
    or neither, the tokens are the same (float32: the kernels are deterministic per row)."""
    import random

    from helios_b200.config import EngineConfig
    from helios_b200.engine.llm import LLMEngine
    from helios_b200.engine.types import SamplingParams

    folder = model_folders[name]
    cfg, _ = read_folder(folder)
    V = cfg["vocab_size"]

    def run(graphs, ahead):
        rng = random.Random(5)
        eng = LLMEngine(EngineConfig(model_dir=str(folder), dtype="float32", block_size=8, num_blocks=36,
                                     max_num_seqs=6, max_num_batched_tokens=48, run_ahead=ahead,
                                     use_cuda_graphs=graphs, watermark=0.0))
        arrivals = []
        for i in range(16):
            prompt = [rng.randrange(V) for _ in range(rng.randint(1, 50))]
            params = SamplingParams(max_tokens=rng.randint(1, 30), temperature=rng.choice([0.0, 0.9]), seed=50 + i)
            arrivals.append((rng.randint(0, 60), f"r{i}", prompt, params))
        arrivals.sort(key=lambda a: a[0])
        done, step = {}, 0
        while arrivals or eng.scheduler.has_work:
            while arrivals and arrivals[0][0] <= step:
                _, rid, prompt, params = arrivals.pop(0)
                eng.add_request(rid, prompt, params)
            for out in eng.step():
                done[out.request_id] = out.token_ids
            step += 1
            assert step < 5000
        captured = [k for k, g in eng.core._graphs.items() if g.graph is not None]
        return done, captured, eng.scheduler.stats.preemptions

    plain, none, _ = run(False, False)
    assert none == [] and len(plain) == 16
    for graphs, ahead in ((True, False), (True, True), (False, True)):
        got, captured, preemptions = run(graphs, ahead)
        assert got == plain, f"graphs={graphs} ahead={ahead}"
        if graphs:
            assert any(s != t for s, t in captured) and any(s == t for s, t in captured)
