"""The persistent decode-step kernel: decode steps of up to eight requests through the
engine with the kernel on, against the plain implementation and against the same steps run
part by part; context slices that are merged, a window, shared slots, captured graphs."""
import pytest
import torch

import plain_model
from conftest import TINY_CONFIGS, assert_logits_close, bf16_round, random_tokens, read_folder

pytestmark = pytest.mark.gpu


def _core(folder, **kw):
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_folder(folder, dtype="bfloat16")
    opts = dict(page_size=16, num_pages=160, max_slots=8, poison_cache=float("nan"))
    opts.update(kw)
    return EngineCore(model, **opts)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", list(TINY_CONFIGS))
def test_decode_steps_of_several_requests_match_the_plain_implementation(model_folders, name, graphs):
    from helios_b200.engine.batch import StepEntry

    cfg, weights = read_folder(model_folders[name])
    w = bf16_round(weights)
    core = _core(model_folders[name], use_cuda_graphs=graphs)
    fused = core.model.plan.fused_steps[0]
    assert fused.ok
    lens = [3, 70, 17, 141, 1, 33, 64, 250][: 8 if name != "tiny_window" else 5]
    n_new = 6
    prompts = [random_tokens(cfg["vocab_size"], n + n_new, 500 + n) for n in lens]
    refs = [plain_model.forward_logits(cfg, w, p) for p in prompts]
    for i, (p, n) in enumerate(zip(prompts, lens)):
        core.step([StepEntry(f"r{i}", p[:n], [])])
    before = fused.steps_run
    for j in range(n_new):
        got = core.step([StepEntry(f"r{i}", [p[n + j]], [0]) for i, (p, n) in enumerate(zip(prompts, lens))])
        want = torch.stack([r[n + j] for r, n in zip(refs, lens)])
        assert_logits_close(got, want, "bfloat16", f"{name}: decode step {j} of {len(lens)} requests")
    # (a captured step is replayed without passing through Python)
    assert fused.steps_run - before >= (3 if graphs else n_new), "the decode steps did not take the fused kernel"
    if graphs:
        assert core._graphs
    from helios_b200.csrc import ops
    ops.check_kernel_errors()


def test_the_fused_step_agrees_with_the_parts_run_one_by_one(model_folders):
    """Same cache contents, same tokens: the two paths differ by rounding only, and both write
    the same keys and values."""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.models import dense_decode_step

    name = "tiny_tiled"
    cfg, _ = read_folder(model_folders[name])
    outs, caches = [], []
    for enabled in (True, False):
        dense_decode_step.ENABLED = enabled
        try:
            core = _core(model_folders[name], use_cuda_graphs=False)
            toks = [random_tokens(cfg["vocab_size"], 90, 7 + i) for i in range(3)]
            for i, t in enumerate(toks):
                core.step([StepEntry(i, t[:80], [])])
            rows = []
            for j in range(80, 90):
                rows.append(core.step([StepEntry(i, [t[j]], [0]) for i, t in enumerate(toks)]).clone())
            outs.append(torch.cat(rows))
            caches.append([s.clone() for s in core.cache.storage])
        finally:
            dense_decode_step.ENABLED = True
    scale = outs[1].abs().max()
    assert (outs[0] - outs[1]).abs().max() <= 0.03 * scale
    for a, b in zip(*caches):
        both = ~(torch.isnan(a.float()) | torch.isnan(b.float()))
        assert torch.equal(torch.isnan(a.float()), torch.isnan(b.float()))          # the same slots were written
        assert (a.float()[both] - b.float()[both]).abs().max() <= 0.05 * b.float()[both].abs().max()


@pytest.mark.parametrize("n_req", [1, 2, 8])
def test_long_contexts_are_cut_into_slices_and_merged(tmp_path, n_req):
    """Head size 64, groups of 7 (the small Qwen's shape), contexts of a thousand keys: one
    request is cut into many slices, eight into few; one far key decides the output."""
    from helios_b200.engine.batch import StepEntry
    from helios_b200.weights import write_model_folder

    cfg = dict(TINY_CONFIGS["tiny_qwen"], hidden_size=128, num_attention_heads=14, num_key_value_heads=2,
               head_dim=64, intermediate_size=208, max_position_embeddings=4096, num_hidden_layers=2)
    folder = write_model_folder(tmp_path / "m", cfg, 9)
    _, weights = read_folder(folder)
    w = bf16_round(weights)
    core = _core(folder, num_pages=8 * 70, use_cuda_graphs=False)
    fused = core.model.plan.fused_steps[0]
    lens = [1000, 513, 40, 999, 257, 1, 700, 64][:n_req]
    prompts = [random_tokens(cfg["vocab_size"], n + 3, 900 + n) for n in lens]
    refs = [plain_model.forward_logits(cfg, w, p) for p in prompts]
    for i, (p, n) in enumerate(zip(prompts, lens)):
        for lo in range(0, n, 256):
            core.step([StepEntry(i, p[lo:min(n, lo + 256)], [])])
    before = fused.steps_run
    for j in range(3):
        got = core.step([StepEntry(i, [p[n + j]], [0]) for i, (p, n) in enumerate(zip(prompts, lens))])
        want = torch.stack([r[n + j] for r, n in zip(refs, lens)])
        assert_logits_close(got, want, "bfloat16", f"{n_req} requests, long contexts, step {j}")
    assert fused.steps_run - before == 3
    from helios_b200.csrc import ops
    ops.check_kernel_errors()


def test_what_the_kernel_does_not_restate_runs_part_by_part(model_folders):
    from helios_b200.engine.batch import StepEntry

    core = _core(model_folders["tiny_llama"], use_cuda_graphs=False)
    fused = core.model.plan.fused_steps[0]
    cfg, _ = read_folder(model_folders["tiny_llama"])
    toks = random_tokens(cfg["vocab_size"], 30, 1)
    core.step([StepEntry("a", toks[:20], [19])])               # a portion: not a decode step
    core.step([StepEntry(f"x{i}", [toks[i]], [0]) for i in range(7)] + [StepEntry("a", [toks[20]], [])])   # a row nobody wants
    assert fused.steps_run == 0
    core.step([StepEntry("a", [toks[21]], [0])])
    assert fused.steps_run == 1
