"""Each request alone and whole: one step over the whole sequence, logits at every
place, against the plain implementation."""
import pytest

from conftest import (TINY_CONFIGS, assert_logits_close, bf16_round, random_tokens, read_folder)
import plain_model

pytestmark = pytest.mark.gpu

LENGTHS = [1, 5, 17, 33, 100]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_whole_sequences(model_folders, name, dtype):
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    folder = model_folders[name]
    cfg, weights = read_folder(folder)
    if dtype == "bfloat16":
        weights = bf16_round(weights)
    model = DecoderModel.from_folder(folder, dtype=dtype)
    core = EngineCore(model, page_size=16, num_pages=16, max_slots=2, poison_cache=float("nan"))
    for i, n in enumerate(LENGTHS):
        toks = random_tokens(cfg["vocab_size"], n, 100 + i)
        logits = core.step([StepEntry(f"r{i}", toks, list(range(n)))])
        core.end(f"r{i}")
        want = plain_model.forward_logits(cfg, weights, toks)
        assert_logits_close(logits, want, dtype, f"{name} n={n}")
    core.cache.check_invariants()
