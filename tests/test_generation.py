"""Generation through the Python entry point and the command line: greedy tokens equal
the plain implementation's, temperature sampling does not depend on the batch, a pool
that is too small preempts and still gives the same tokens, long decoding, the first
tokens of a sequence."""
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, TINY_CONFIGS, bf16_round, random_tokens, read_folder
import plain_model

pytestmark = pytest.mark.gpu


def _engine(folder, **kw):
    from helios_b200.config import EngineConfig
    from helios_b200.engine.llm import LLMEngine

    opts = dict(model_dir=str(folder), dtype="float32", kv_cache_bytes=1 << 24, block_size=16)
    opts.update(kw)
    return LLMEngine(EngineConfig(**opts))


def _check_greedy(cfg, weights, prompt, got, dtype):
    """Every generated token is the plain implementation's argmax given the tokens before
    it; in bfloat16 a near-tie may fall the other way, but only within rounding."""
    toks = list(prompt)
    for t in got:
        logits = plain_model.forward_logits(cfg, weights, toks)[-1]
        best = int(torch.argmax(logits))
        if t != best:
            assert dtype == "bfloat16", f"token {t} instead of {best} after {len(toks)} tokens"
            assert float(logits[best] - logits[t]) <= 0.03 * float(logits.abs().max())
        toks.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_greedy_generation_matches_the_plain_implementation(model_folders, name, dtype):
    from helios_b200 import LLM, SamplingParams

    cfg, weights = read_folder(model_folders[name])
    w = bf16_round(weights) if dtype == "bfloat16" else weights
    prompts = [random_tokens(cfg["vocab_size"], n, 40 + n) for n in (1, 5, 17, 33)]
    llm = LLM(str(model_folders[name]), dtype=dtype, kv_cache_bytes=1 << 24, max_num_batched_tokens=24)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(max_tokens=16))
    assert [o.request_id for o in outs] == [f"batch-{i}" for i in range(4)]
    for prompt, out in zip(prompts, outs):
        assert out.completion_tokens == 16 and out.finish_reason.value == "length"
        assert out.prompt_tokens == len(prompt)
        _check_greedy(cfg, w, prompt, out.token_ids, dtype)


def test_same_tokens_whole_token_by_token_in_chunks_and_mixed(model_folders):
    """python/helios tests/parity/test_parity.py:273-304 in spirit: however the scheduler cuts
    and batches, greedy float32 tokens are the same."""
    from helios_b200.engine.types import SamplingParams

    folder = model_folders["tiny_llama"]
    cfg, _ = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 70 + n) for n in (1, 5, 17, 33)]
    runs = []
    for opts in (dict(max_num_batched_tokens=2048), dict(max_num_batched_tokens=7),
                 dict(max_num_batched_tokens=1), dict(max_num_seqs=1), dict(use_cuda_graphs=False),
                 dict(block_size=8, max_num_batched_tokens=5)):
        eng = _engine(folder, **opts)
        outs = eng.generate(prompts, SamplingParams(max_tokens=16))
        runs.append([o.token_ids for o in outs])
        eng.scheduler.check_invariants()
    assert all(r == runs[0] for r in runs[1:])


def test_staggered_arrivals_and_seeded_sampling_do_not_depend_on_the_batch(model_folders):
    from helios_b200.engine.types import SamplingParams

    folder = model_folders["tiny_qwen"]
    cfg, _ = read_folder(folder)
    lengths = (2, 9, 31, 64, 100, 3)
    prompts = [random_tokens(cfg["vocab_size"], n, 90 + n) for n in lengths]
    params = [SamplingParams(max_tokens=24, temperature=0.8, seed=1000 + i) for i in range(6)]

    def alone(i):
        eng = _engine(folder)
        eng.add_request("r", prompts[i], params[i])
        return eng.run_until_complete()[0].token_ids

    singles = [alone(i) for i in range(6)]
    for budget in (1, 13, 64):
        eng = _engine(folder, max_num_batched_tokens=budget, max_num_seqs=4)
        done = {}
        pending = list(range(6))
        steps = 0
        while pending or eng.scheduler.has_work:
            if pending and steps % 3 == 0:                      # a new request every third step
                i = pending.pop(0)
                eng.add_request(f"r{i}", prompts[i], params[i])
            for out in eng.step():
                done[out.request_id] = out.token_ids
            steps += 1
            assert steps < 5000
        assert [done[f"r{i}"] for i in range(6)] == singles, f"budget {budget}"
    # another seed gives other tokens
    eng = _engine(folder)
    eng.add_request("other", prompts[3], SamplingParams(max_tokens=24, temperature=0.8, seed=5))
    assert eng.run_until_complete()[0].token_ids != singles[3]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("slots", [8, 3])
def test_running_ahead_of_the_host_changes_no_token(model_folders, dtype, graphs, slots):
    """The next decode step is launched with token ids that are still on the device; the
    outputs equal those of an engine that reads every token first.  Requests stop at
    different steps (stop tokens found one step late, lengths known ahead), and one arrives
    in the middle.  With three slots some requests wait while the others decode ahead."""
    from helios_b200.engine.types import SamplingParams

    folder = model_folders["tiny_llama"]
    cfg, _ = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 40 + n) for n in (7, 33, 64, 18, 5)]

    def run(ahead, stops):
        eng = _engine(folder, dtype=dtype, run_ahead=ahead, use_cuda_graphs=graphs, max_num_seqs=slots)
        params = [SamplingParams(max_tokens=30 + 9 * i, temperature=0.7 if i % 2 else 0.0, seed=77 + i,
                                 stop_token_ids=stops[i]) for i in range(5)]
        done, steps = {}, 0
        for i in range(4):
            eng.add_request(f"r{i}", prompts[i], params[i])
        while eng.scheduler.has_work:
            if steps == 20:
                eng.add_request("r4", prompts[4], params[4])
            for out in eng.step():
                done[out.request_id] = (out.token_ids, out.finish_reason)
            steps += 1
            assert steps < 2000
        eng.scheduler.check_invariants()
        assert all(p.num_free == p.num_pages for p in eng.core.cache.pools)
        return done, eng.steps_ahead

    free, _ = run(False, [[]] * 5)
    # stop two requests on a token they are known to make in the middle of their output
    stops = [[free["r0"][0][11]], [], [free["r2"][0][25]], [], []]
    want, none_ahead = run(False, stops)
    got, n_ahead = run(True, stops)
    assert none_ahead == 0 and n_ahead > 40
    assert got == want
    assert len(want["r0"][0]) <= 12 and len(want["r2"][0]) <= 26


@pytest.mark.parametrize("dtype", ["float32"])
def test_output_survives_preemption_with_outputs_already_made(model_folders, dtype):
    """The reference's own test only ever preempts sequences without outputs
    (tests/parity/test_parity.py:480-519); here the pool is so small that running requests
    are preempted in mid-decode and must still give the tokens of an undisturbed run."""
    from helios_b200.engine.types import SamplingParams

    folder = model_folders["tiny_llama"]
    cfg, _ = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 20 + n) for n in (20, 21, 22, 23)]
    roomy = _engine(folder, num_blocks=200, block_size=4)
    want = [o.token_ids for o in roomy.generate(prompts, SamplingParams(max_tokens=40))]
    assert roomy.scheduler.stats.preemptions == 0
    tight = _engine(folder, num_blocks=34, block_size=4, watermark=0.0)
    got = [o.token_ids for o in tight.generate(prompts, SamplingParams(max_tokens=40))]
    assert tight.scheduler.stats.preemptions >= 1
    assert got == want
    tight.scheduler.check_invariants()
    assert all(p.num_used == 0 for p in tight.core.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_window", "tiny_tiled"])
def test_long_decoding(model_folders, name, dtype):
    """Hundreds of decode steps: across many pages, past the window, through captured
    graphs; compared position by position with the plain implementation's logits."""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel
    from conftest import assert_logits_close

    cfg, weights = read_folder(model_folders[name])
    w = bf16_round(weights) if dtype == "bfloat16" else weights
    toks = random_tokens(cfg["vocab_size"], 420, 9)
    want = plain_model.forward_logits(cfg, w, toks)
    core = EngineCore(DecoderModel.from_folder(model_folders[name], dtype=dtype), page_size=16,
                      num_pages=28, max_slots=2, poison_cache=float("nan"))
    got = [core.step([StepEntry("a", toks[:20], [19])])]
    for i in range(20, len(toks)):
        got.append(core.step([StepEntry("a", [toks[i]], [0])]).clone())
    assert_logits_close(torch.cat(got), want[19:], dtype, f"{name} long decode")
    assert core._graphs, "decode steps should have run as captured graphs"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(model_folders, dtype):
    """Positions 0, 1, 2: an empty cache, one key, the first page's first slots."""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel
    from conftest import assert_logits_close

    for name in TINY_CONFIGS:
        cfg, weights = read_folder(model_folders[name])
        w = bf16_round(weights) if dtype == "bfloat16" else weights
        toks = random_tokens(cfg["vocab_size"], 4, 3)
        want = plain_model.forward_logits(cfg, w, toks)
        core = EngineCore(DecoderModel.from_folder(model_folders[name], dtype=dtype), page_size=16,
                          num_pages=4, max_slots=2, poison_cache=float("nan"))
        one_by_one = torch.cat([core.step([StepEntry("a", [t], [0])]).clone() for t in toks])
        assert_logits_close(one_by_one, want, dtype, f"{name} first tokens one by one")
        core.end("a")
        pair = torch.cat([core.step([StepEntry("b", toks[:2], [0, 1])]),
                          core.step([StepEntry("b", toks[2:], [0, 1])])])
        assert_logits_close(pair, want, dtype, f"{name} first tokens in pairs")


def test_stop_token_and_max_model_len(model_folders):
    from helios_b200.engine.types import SamplingParams

    folder = model_folders["tiny_llama"]
    cfg, weights = read_folder(folder)
    prompt = random_tokens(cfg["vocab_size"], 9, 1)
    free = _engine(folder).generate([prompt], SamplingParams(max_tokens=12))[0].token_ids
    stop = free[4]
    out = _engine(folder).generate([prompt], SamplingParams(max_tokens=12, stop_token_ids=[stop]))[0]
    cut = free.index(stop) + 1
    assert out.token_ids == free[:cut] and out.finish_reason.value == "stop"
    out = _engine(folder, max_model_len=14).generate([prompt], SamplingParams(max_tokens=50))[0]
    assert len(prompt) + out.completion_tokens == 14 and out.finish_reason.value == "length"
    with pytest.raises(ValueError):
        _engine(folder, max_model_len=8).add_request("x", prompt)
    with pytest.raises(ValueError):
        _engine(folder).add_request("x", [cfg["vocab_size"]])


def test_command_line(model_folders, tmp_path):
    from helios_b200.weights import write_model_folder

    folder = model_folders["tiny_llama"]
    cfg, weights = read_folder(folder)
    run = lambda *a: subprocess.run([sys.executable, "-m", "helios_b200.cli", *a], cwd=str(ROOT),
                                    capture_output=True, text=True, timeout=300)
    # the same weights in a folder without a tokenizer: the ids themselves are printed
    bare = write_model_folder(tmp_path / "bare", TINY_CONFIGS["tiny_llama"], 11, tokenizer=False)
    out = run("generate", "--model", str(bare), "--prompt-ids", "5,17,3", "8,8", "--max-tokens", "5",
              "--dtype", "float32", "--kv-mb", "16")
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    assert lines[0] == "--- batch-0 ---" and lines[2] == "[5 tokens, finish=length]"
    assert lines[3] == "--- batch-1 ---"
    for line, prompt in ((lines[1], [5, 17, 3]), (lines[4], [8, 8])):
        assert line.startswith("(token ids: [") and line.endswith("])"), line
        ids = [int(t) for t in line[len("(token ids: ["):-2].split(",")]
        assert ids == plain_model.greedy_generate(cfg, weights, prompt, 5)
    # with the byte tokenizer the text form is printed; its bytes are the same tokens
    text = run("generate", "--model", str(folder), "--prompt-ids", "5,17,3", "--max-tokens", "5",
               "--dtype", "float32", "--kv-mb", "16")
    assert text.returncode == 0 and "[5 tokens" in text.stdout
    text = run("generate", "--model", str(folder), "--prompt", "hi", "--max-tokens", "3", "--dtype", "float32",
               "--kv-mb", "16")
    assert text.returncode == 0 and "[3 tokens" in text.stdout
    info = run("info", "--model", str(folder))
    assert info.returncode == 0 and "LlamaForCausalLM" in info.stdout
    assert "2 x PreNormBlock(RMSNorm, GQAAttention, RMSNorm, SwiGLU)" in info.stdout
    n_params = sum(t.numel() for t in weights.values())
    assert f"{n_params:,} parameters" in info.stdout and "bytes a page" in info.stdout
    toy = run("make-toy-model", "--out", str(tmp_path / "toy"), "--arch", "qwen2", "--tie", "--layers", "1")
    assert toy.returncode == 0 and (tmp_path / "toy" / "model.safetensors").exists()
    toy_cfg, toy_w = read_folder(tmp_path / "toy")
    assert toy_cfg["architectures"] == ["Qwen2ForCausalLM"] and "lm_head.weight" not in toy_w
    assert "model.layers.0.self_attn.q_proj.bias" in toy_w
    bad = run("generate", "--model", str(tmp_path / "nowhere"), "--prompt-ids", "1")
    assert bad.returncode == 2 and bad.stderr.startswith("error:")
    bad = run("make-toy-model", "--out", str(tmp_path / "toy2"), "--arch", "mamba")
    assert bad.returncode == 2 and "known:" in bad.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_whose_every_layer_has_a_window_runs_past_its_pool(tmp_path, dtype):
    """Every layer sees only the last 24 keys, so the cache holds window + portion whatever
    the length: a prompt three times the pool is admitted, fed portion by portion (pages
    taken per portion and given back behind the window), and generates the tokens of a roomy
    pool; its logits are the plain implementation's."""
    from conftest import assert_logits_close
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.types import SamplingParams
    from helios_b200.weights import write_model_folder

    cfg = dict(TINY_CONFIGS["tiny_window"], sliding_window=24, max_window_layers=0, max_position_embeddings=4096)
    folder = write_model_folder(tmp_path / "all_window", cfg, 5)
    _, weights = read_folder(folder)
    w = bf16_round(weights) if dtype == "bfloat16" else weights
    page, pages = 8, 12                                   # 96 tokens of cache
    prompts = [random_tokens(cfg["vocab_size"], n, 70 + n) for n in (300, 41)]
    tight = _engine(folder, dtype=dtype, num_blocks=pages, block_size=page, max_num_batched_tokens=16,
                    watermark=0.0, max_num_seqs=2)
    assert tight.max_model_len == 4096                    # not the pool's 96 tokens
    got = tight.generate(prompts, SamplingParams(max_tokens=12))
    assert [o.finish_reason.value for o in got] == ["length", "length"]
    tight.scheduler.check_invariants()
    assert all(p.num_used == 0 for p in tight.core.cache.pools)
    roomy = _engine(folder, dtype=dtype, num_blocks=200, block_size=page, max_num_batched_tokens=16)
    want = roomy.generate(prompts, SamplingParams(max_tokens=12))
    if dtype == "float32":
        assert [o.token_ids for o in got] == [o.token_ids for o in want]
    for prompt, out in zip(prompts, got):
        _check_greedy(cfg, w, prompt, out.token_ids, dtype)
    # the same through the step function: portions of 16, logits wanted at the end of each
    core = tight.core
    toks = prompts[0]
    plain = plain_model.forward_logits(cfg, w, toks)
    rows, places = [], []
    for lo in range(0, len(toks), 16):
        part = toks[lo:lo + 16]
        rows.append(core.step([StepEntry("again", part, [0, len(part) - 1])]).clone())
        places += [lo, lo + len(part) - 1]
        assert max(p.num_used for p in core.cache.pools) <= pages
    assert_logits_close(torch.cat(rows), plain[places], dtype, "all-window model, portions of 16")
    core.end("again")
