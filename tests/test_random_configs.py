"""Configurations drawn at random (head sizes in steps of 16 up to 256, any number of heads
and groups, widths and vocabularies that are no power of two, windows on some layers,
scaled rotary frequencies, bias, tied head): the engine against the plain implementation
with the requests cut three ways, in float32 and bfloat16.  A configuration the kernels
do not take must be refused with a clear error, never give a wrong result."""
import random

import pytest

from conftest import bf16_round, random_tokens, read_folder
import plain_model
import trace_util as tu

pytestmark = pytest.mark.gpu


def draw_config(seed, scale, head_dims=(16, 32, 48, 64, 80, 96, 112, 128, 144, 160, 192, 256)):
    rng = random.Random(seed)
    head_dim = rng.choice(list(head_dims))
    kv_heads = rng.choice([1, 2, 3, 4, 5])
    heads = kv_heads * rng.choice([1, 2, 3, 4, 6, 7, 8])
    layers = rng.randint(1, 4 if scale == 1 else 2)
    qwen = rng.random() < 0.5
    cfg = {
        "architectures": ["Qwen2ForCausalLM" if qwen else "LlamaForCausalLM"],
        "model_type": "qwen2" if qwen else "llama",
        "vocab_size": rng.randint(40, 1500 * scale),
        "hidden_size": 8 * rng.randint(2 * scale, 30 * scale),
        "intermediate_size": 8 * rng.randint(2 * scale, 50 * scale),
        "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "head_dim": head_dim, "max_position_embeddings": 4096,
        "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-6, 2e-5]),
        "rope_theta": rng.choice([10000.0, 500000.0, 1e6]),
        "tie_word_embeddings": rng.random() < 0.5, "hidden_act": "silu", "torch_dtype": "float32",
        "attention_bias": rng.random() < 0.5,
    }
    if rng.random() < 0.4:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]),
                               "low_freq_factor": 1.0, "high_freq_factor": rng.choice([2.0, 4.0]),
                               "original_max_position_embeddings": rng.choice([16, 64, 256])}
    if rng.random() < 0.5 and qwen:           # a Llama configuration with a window is refused
        cfg["sliding_window"] = rng.randint(3, 90)
        cfg["layer_types"] = [rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)]
    return cfg, rng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed,scale", [(s, 1) for s in range(10)] + [(2000 + s, 8) for s in range(4)])
def test_a_random_configuration_matches_the_plain_implementation(tmp_path, seed, scale, dtype):
    cfg, rng = draw_config(seed, scale)
    _compare(tmp_path, cfg, rng, seed, scale, dtype)


@pytest.mark.parametrize("seed", range(3000, 3008))
def test_random_configurations_on_the_tensor_memory_attention_kernels(tmp_path, seed, monkeypatch):
    """Head sizes 64 and 128 in bfloat16 run their prompt portions on the tcgen05 attention
    kernels; here also the kernel with two query tiles per block, which otherwise waits for
    steps of many blocks."""
    from helios_b200.csrc import ops

    monkeypatch.setattr(ops, "ATTENTION_PAIR_MIN_BLOCKS", 1 if seed % 2 == 0 else 10 ** 6)
    before = ops.launch_count
    cfg, rng = draw_config(seed, 1, head_dims=(64, 128))
    _compare(tmp_path, cfg, rng, seed, 1, "bfloat16", page_sizes=(8, 16, 32))
    assert ops.launch_count > before


@pytest.mark.parametrize("seed", range(4000, 4008))
def test_random_configurations_with_the_norms_inside_the_products(tmp_path, seed, monkeypatch):
    """Steps of few tokens run without RMSNorm launches: the products add into the residual,
    leave the next norm's input and apply 1 / rms to their accumulators (here at sizes that
    are no multiples of a tile, with bias and windows, and with the limit raised from 16 to
    the 32 tokens the epilogues take), and decode attention rotates and stores the new token
    itself."""
    from helios_b200.csrc import ops
    monkeypatch.setattr(ops, "DEFERRED_NORM_TOKENS", ops.DEFERRED_NORM_MOST if seed % 2 else 16)
    cfg, rng = draw_config(seed, 8, head_dims=(32, 64, 96, 128, 48))
    _compare(tmp_path, cfg, rng, seed, 8, "bfloat16")


def _compare(tmp_path, cfg, rng, seed, scale, dtype, page_sizes=(8, 16, 32)):
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel
    from helios_b200.weights import write_model_folder

    folder = write_model_folder(tmp_path / "model", cfg, seed)
    cfg, weights = read_folder(folder)
    lengths = [rng.randint(2, 150 if scale == 1 else 300) for _ in range(6)]
    reqs = {f"q{i}": random_tokens(cfg["vocab_size"], n, seed * 100 + i) for i, n in enumerate(lengths)}
    w = bf16_round(weights) if dtype == "bfloat16" else weights
    plain = {rid: plain_model.forward_logits(cfg, w, toks) for rid, toks in reqs.items()}
    model = DecoderModel.from_folder(folder, dtype=dtype)
    for kind in ("mixed", "decode", "portions"):
        tb = tu.TraceBuilder()
        if kind == "mixed":
            tu.mixed(tb, reqs, seed=seed)
        elif kind == "decode":
            for rid, toks in list(reqs.items())[:3]:
                tu.prefill_then_decode(tb, rid, toks, n_decode=32)
        else:
            for rid, toks in list(reqs.items())[3:]:
                tu.portions(tb, rid, toks, [rng.choice([2, 3, 7, 16, 31]) for _ in range(4)])
        page = rng.choice(list(page_sizes))
        core = EngineCore(model, page_size=page, num_pages=-(-tb.live_tokens_peak // page), max_slots=4,
                          poison_cache=float("nan"))
        tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{cfg} {kind}")
        assert all(p.num_used == 0 for p in core.cache.pools)
