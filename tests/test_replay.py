"""Replay of the same requests cut in different ways, in float32 and bfloat16,
against the plain implementation: whole; most in one step and the last 32 tokens
one by one; portions of changing size down to two tokens; and mixed, up to four
live requests with so few pages that they are used again.  Once per
configuration and dtype the whole set also goes through ``bin/trace_run``."""
import pytest

from conftest import TINY_CONFIGS, bf16_round, random_tokens, read_folder
import plain_model
import trace_util as tu

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def _plain(cfg, weights, dtype, requests):
    w = bf16_round(weights) if dtype == "bfloat16" else weights
    return {rid: plain_model.forward_logits(cfg, w, toks) for rid, toks in requests.items()}


def _core(folder, dtype, max_tokens, page_size=16, max_slots=4):
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_folder(folder, dtype=dtype)
    return EngineCore(model, page_size=page_size, num_pages=-(-max_tokens // page_size),
                      max_slots=max_slots, poison_cache=float("nan"))


def _requests(cfg, lengths, seed):
    return {f"q{i}": random_tokens(cfg["vocab_size"], n, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_prefill_then_decode_one_by_one(model_folders, name, dtype):
    cfg, weights = read_folder(model_folders[name])
    reqs = _requests(cfg, [33, 70, 129], 500)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.prefill_then_decode(tb, rid, toks, n_decode=32)
    core = _core(model_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_portions_of_changing_size(model_folders, name, dtype):
    cfg, weights = read_folder(model_folders[name])
    reqs = _requests(cfg, [64, 97, 50], 600)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    sizes = [[7], [2, 31, 3, 16, 2, 17], [13, 2, 1, 5]]
    for (rid, toks), sz in zip(reqs.items(), sizes):
        tu.portions(tb, rid, toks, sz)
    core = _core(model_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} portions")


@pytest.mark.parametrize("page_size", [16, 8])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_mixed_with_page_reuse(model_folders, name, dtype, page_size):
    cfg, weights = read_folder(model_folders[name])
    reqs = _requests(cfg, [70, 45, 130, 33, 90, 64, 17, 101], 700)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=7)
    core = _core(model_folders[name], dtype, tb.live_tokens_peak, page_size=page_size)
    total_pages = sum(-(-len(t) // page_size) for t in reqs.values())
    assert total_pages > core.cache.pools[0].num_pages, "the pool must be too small to avoid reuse"
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} mixed")
    assert all(p.num_used == 0 for p in core.cache.pools)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_through_trace_run(model_folders, name, dtype, tmp_path):
    """Everything above in one trace through the program a user runs."""
    cfg, weights = read_folder(model_folders[name])
    reqs = _requests(cfg, [40, 75, 66, 52, 81, 38], 800)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    ids = list(reqs)
    tu.whole(tb, ids[0], reqs[ids[0]])
    tu.prefill_then_decode(tb, ids[1], reqs[ids[1]], 32)
    tu.portions(tb, ids[2], reqs[ids[2]], [2, 9, 4, 2, 30])
    tu.mixed(tb, {r: reqs[r] for r in ids[3:]}, seed=3, max_live=3)
    got = tu.run_trace_run(model_folders[name], dtype, tb, tmp_path / "out", tb.live_tokens_peak,
                           cfg["vocab_size"])
    tu.check(tb, got, plain, dtype, f"{name} trace_run")
