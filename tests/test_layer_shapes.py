"""One layer with the layer sizes of Llama-3.1-8B (width 4096, 32 query / 8 KV heads of 128,
feed-forward 14336; small vocabulary) in bfloat16 against the plain implementation: the
tile shapes, split counts and kernel choices of the real sizes, which the tiny
configurations never reach.  A prompt long enough for the two-SM products and the tcgen05
attention, the same prompt in portions, single decoded tokens, and a batch of eight."""
import pytest
import torch

import plain_model
from conftest import assert_logits_close, random_tokens
from test_parts import _export

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 1024, "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 1,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "attention_bias": False, "tie_word_embeddings": False, "hidden_act": "silu",
}


def test_one_layer_of_the_benchmarks_sizes_matches_the_plain_implementation():
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_config(CONFIG, seed=5, dtype="bfloat16")
    weights = _export(model.plan)
    core = EngineCore(model, page_size=16, num_pages=400, max_slots=10)
    n = 1100
    toks = random_tokens(CONFIG["vocab_size"], n + 3, 77)
    want = plain_model.forward_logits(CONFIG, weights, toks, dtype=torch.float32)
    places = [0, 1, 127, 128, 129, 500, 1023, 1024, n - 2, n - 1]

    # whole prompt in one step, then three tokens one by one
    got = core.step([StepEntry("whole", toks[:n], places)])
    assert_logits_close(got, want[places], "bfloat16", "1,100 tokens in one step")
    for i in range(3):
        got = core.step([StepEntry("whole", [toks[n + i]], [0])])
        assert_logits_close(got, want[n + i:n + i + 1], "bfloat16", f"decoded token {i}")
    core.end("whole")

    # the same prompt in portions of 700 and 400 tokens (other kernels for the products)
    core.step([StepEntry("cut", toks[:700], [])])
    got = core.step([StepEntry("cut", toks[700:n], [0, n - 701])])
    assert_logits_close(got, want[[700, n - 1]], "bfloat16", "portions of 700 and 400 tokens")
    core.end("cut")

    # eight requests decoding together (twice: the second step of a batch size is a captured graph)
    prompts = [random_tokens(CONFIG["vocab_size"], 20 + 9 * i, 100 + i) for i in range(8)]
    refs = [plain_model.forward_logits(CONFIG, weights, p, dtype=torch.float32) for p in prompts]
    core.step([StepEntry(f"b{i}", p[:-3], []) for i, p in enumerate(prompts)])
    for back in (3, 2, 1):
        got = core.step([StepEntry(f"b{i}", [p[-back]], [0]) for i, p in enumerate(prompts)])
        want8 = torch.stack([r[len(p) - back] for r, p in zip(refs, prompts)])
        assert_logits_close(got, want8, "bfloat16", f"batch of eight, {back} from the end")
    from helios_b200.csrc import ops
    ops.check_kernel_errors()


def _close_f32(got, want, what):
    """Sums of 4,096 and 14,336 float32 products, and logits that reach 5 where the tiny
    models' stay near 1: the error is judged against the row's largest |logit|, at 2e-5 of it
    (which is what the tiny models' absolute 2e-5 amounts to for them)."""
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    rel = ((got - want).abs() / want.abs().amax(dim=-1, keepdim=True)).max().item()
    assert rel <= 2e-5, f"{what}: max |err| / max |logit| = {rel:.3e} > 2e-5"


def test_one_layer_of_the_benchmarks_sizes_in_float32():
    """The 32-bit path at the real widths: the FMA product's grid at 4096 x 14336, the generic
    attention kernel at 32 heads of 128; whole, in portions, and eight requests decoding."""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_config(CONFIG, seed=6, dtype="float32")
    weights = _export(model.plan)
    core = EngineCore(model, page_size=16, num_pages=200, max_slots=10)
    n = 300
    toks = random_tokens(CONFIG["vocab_size"], n + 2, 78)
    want = plain_model.forward_logits(CONFIG, weights, toks)
    places = [0, 1, 127, 128, 129, n - 1]
    got = core.step([StepEntry("whole", toks[:n], places)])
    _close_f32(got, want[places], "300 tokens in one step, float32")
    for i in range(2):
        got = core.step([StepEntry("whole", [toks[n + i]], [0])])
        _close_f32(got, want[n + i:n + i + 1], f"decoded token {i}, float32")
    core.end("whole")
    core.step([StepEntry("cut", toks[:131], [])])
    got = core.step([StepEntry("cut", toks[131:n], [0, n - 132])])
    _close_f32(got, want[[131, n - 1]], "portions of 131 and 169 tokens, float32")
    core.end("cut")
    prompts = [random_tokens(CONFIG["vocab_size"], 12 + 5 * i, 200 + i) for i in range(8)]
    refs = [plain_model.forward_logits(CONFIG, weights, p) for p in prompts]
    core.step([StepEntry(f"b{i}", p[:-3], []) for i, p in enumerate(prompts)])
    for back in (3, 2, 1):
        got = core.step([StepEntry(f"b{i}", [p[-back]], [0]) for i, p in enumerate(prompts)])
        want8 = torch.stack([r[len(p) - back] for r, p in zip(refs, prompts)])
        _close_f32(got, want8, f"batch of eight, {back} from the end, float32")


@pytest.mark.parametrize("graphs", [False, True])
def test_a_long_portion_beside_decoded_tokens_at_the_benchmarks_sizes(graphs):
    """A mixed step at the real widths: 700 tokens of one prompt beside six requests that decode,
    three times over (with graphs: kernel by kernel, on the graph's buffers, replayed)."""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_config(CONFIG, seed=5, dtype="bfloat16")
    weights = _export(model.plan)
    core = EngineCore(model, page_size=16, num_pages=400, max_slots=10, use_cuda_graphs=graphs)
    prompts = [random_tokens(CONFIG["vocab_size"], 30 + 21 * i, 300 + i) for i in range(6)]
    refs = [plain_model.forward_logits(CONFIG, weights, p, dtype=torch.float32) for p in prompts]
    core.step([StepEntry(f"d{i}", p[:-3], []) for i, p in enumerate(prompts)])
    for rep in range(3):
        long = random_tokens(CONFIG["vocab_size"], 800, 400 + rep)
        ref_long = plain_model.forward_logits(CONFIG, weights, long, dtype=torch.float32)
        back = 3 - rep
        got = core.step([StepEntry(f"long{rep}", long[:700], [699])]
                        + [StepEntry(f"d{i}", [p[-back]], [0]) for i, p in enumerate(prompts)]).clone()
        want = torch.stack([ref_long[699]] + [r[len(p) - back] for r, p in zip(refs, prompts)])
        assert_logits_close(got, want, "bfloat16", f"700 tokens beside six decoded, run {rep}")
        got = core.step([StepEntry(f"long{rep}", long[700:], [99])])
        assert_logits_close(got, ref_long[799:800], "bfloat16", f"the rest of the long prompt, run {rep}")
        core.end(f"long{rep}")
    from helios_b200.csrc import ops
    ops.check_kernel_errors()


@pytest.mark.parametrize("n", [32, 33, 128, 192, 257, 400])
def test_a_portion_on_either_side_of_the_library_boundary(n):
    """Up to 32 tokens the products run on this package's decode kernel, from 33 to 1,536 the
    plain ones go to the library: a request's bfloat16 numbers are not bit-equal across that
    line, but either side must match the plain model.  (The SwiGLU product changes sides at
    129, 257 and 384 tokens.)"""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_config(CONFIG, seed=5, dtype="bfloat16")
    weights = _export(model.plan)
    core = EngineCore(model, page_size=16, num_pages=64, max_slots=2)
    toks = random_tokens(CONFIG["vocab_size"], n, 79)
    want = plain_model.forward_logits(CONFIG, weights, toks, dtype=torch.float32)
    places = [0, 1, n // 2, n - 1]
    got = core.step([StepEntry("p", toks, places)])
    assert_logits_close(got, want[places], "bfloat16", f"a portion of {n} tokens")


SMALL = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 1000, "hidden_size": 896, "intermediate_size": 4864, "num_hidden_layers": 2,
    "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "hidden_act": "silu",
}


def test_two_layers_of_the_small_models_sizes_across_the_kernel_choices():
    """Qwen2.5-0.5B layer sizes: steps of up to 16 tokens run the tensor-memory products with
    the norms in their epilogues, up to 32 with norm launches, beyond that the library's
    products (small weight matrices); every
    side of each line against the plain implementation, as portions and as batches of
    requests that decode."""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_config(SMALL, seed=8, dtype="bfloat16")
    weights = _export(model.plan)
    core = EngineCore(model, page_size=16, num_pages=400, max_slots=40)
    toks = random_tokens(SMALL["vocab_size"], 260, 80)
    want = plain_model.forward_logits(SMALL, weights, toks, dtype=torch.float32)
    lo = 0
    for n in (16, 17, 32, 33, 64, 98):
        got = core.step([StepEntry("p", toks[lo:lo + n], [0, n - 1])])
        assert_logits_close(got, want[[lo, lo + n - 1]], "bfloat16", f"portion of {n} tokens at {lo}")
        lo += n
    core.end("p")
    for batch in (8, 16, 17, 33):
        prompts = [random_tokens(SMALL["vocab_size"], 9 + 3 * i, 600 + i) for i in range(batch)]
        refs = [plain_model.forward_logits(SMALL, weights, p, dtype=torch.float32) for p in prompts]
        core.step([StepEntry(f"b{batch}_{i}", p[:-2], []) for i, p in enumerate(prompts)])
        for back in (2, 1):
            got = core.step([StepEntry(f"b{batch}_{i}", [p[-back]], [0]) for i, p in enumerate(prompts)])
            wantb = torch.stack([r[len(p) - back] for r, p in zip(refs, prompts)])
            assert_logits_close(got, wantb, "bfloat16", f"{batch} requests decoding, {back} from the end")
        for i in range(batch):
            core.end(f"b{batch}_{i}")
    from helios_b200.csrc import ops
    ops.check_kernel_errors()
