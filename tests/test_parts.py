"""Each part of a layer alone against the plain function it stands for, and what the
part interfaces promise: a model assembled from a list that names a layer twice or lets
a layer read another layer's cache, and a toy mixer with state of its own, defined here,
registered, built and stepped without touching the package's files."""
import math

import pytest
import torch

import plain_model
from conftest import TINY_LLAMA, assert_logits_close, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _ctx(entries_tokens, dtype, page_size=8, num_pages=64):
    """A StepContext over fresh requests without a model: a bare cache layout."""
    from helios_b200.cache import CacheLayout, GroupLayout
    from helios_b200.engine.batch import StepEntry, build_context

    lay = CacheLayout([GroupLayout(None, num_pages)], page_size, max_slots=8)
    entries = []
    for i, toks in enumerate(entries_tokens):
        lay.admit(i)
        lay.extend(i, len(toks))
        entries.append(StepEntry(i, toks, list(range(len(toks)))))
    return build_context(entries, lay, dtype, DEV), lay


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from helios_b200.parts import RMSNorm

    g = torch.Generator().manual_seed(0)
    norm = RMSNorm(200, 3e-6)
    assert norm.weight_specs()["weight"].shape == (200,)
    w = 1 + 0.1 * torch.randn(200, generator=g)
    norm.bind({"weight": w.to(DEV)})
    x = torch.randn(11, 200, generator=g).to(dtype)
    tol = dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(norm.forward(x.to(DEV)).cpu().double(),
                               plain_model.rms_norm(x.double(), w.double(), 3e-6), **tol)


def test_rotary_part_against_the_plain_tables():
    from helios_b200.config import DenseDecoderConfig
    from helios_b200.parts import RotaryEncoding

    cfg = DenseDecoderConfig.from_hf(TINY_LLAMA)
    rope = RotaryEncoding(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling)
    want = plain_model.rope_inv_freq(cfg.head_dim, TINY_LLAMA["rope_theta"], TINY_LLAMA["rope_scaling"])
    torch.testing.assert_close(rope.inv_freq64, want, atol=0, rtol=1e-14)
    ctx, _ = _ctx([[1, 2, 3], [4] * 70], torch.float32)
    rope.prepare(ctx)
    pos = torch.tensor([0, 1, 2] + list(range(70)), dtype=torch.float64)
    torch.testing.assert_close(ctx.rotary_cos.cpu().double(), (pos[:, None] * want[None]).cos(), atol=1e-7, rtol=0)
    assert ctx.rotary_sin.shape == (73, cfg.head_dim // 2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,bias,window", [(4, 2, 16, False, None), (6, 1, 32, True, 20), (5, 5, 48, True, None)])
def test_attention_part_alone(dtype, nh, nkv, hd, bias, window):
    """The mixer with its projections, rotation, cache write and attention, for two
    requests in one batch, against the plain functions on whole sequences."""
    from helios_b200.parts import GQAAttention, LayerCache, RotaryEncoding

    H, page = 72, 8
    g = torch.Generator().manual_seed(nh * hd)
    attn = GQAAttention(H, nh, nkv, hd, 1 / math.sqrt(hd), bias, window=window)
    specs = attn.weight_specs()
    assert ("q_proj.bias" in specs) == bias
    tensors = {k: torch.randn(s.shape, generator=g) * (0.1 if len(s.shape) == 2 else 0.5) for k, s in specs.items()}
    if dtype == torch.bfloat16:
        tensors = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in tensors.items()}
    attn.bind({k: v.to(DEV, dtype if v.dim() == 2 else torch.float32) for k, v in tensors.items()})
    lens = [37, 5]
    ctx, lay = _ctx([[0] * n for n in lens], dtype, page_size=page)
    rope = RotaryEncoding(hd, 10000.0)
    rope.prepare(ctx)
    x = torch.randn(sum(lens), H, generator=g)
    if dtype == torch.bfloat16:
        x = x.to(torch.bfloat16).float()
    spec = attn.cache_spec()
    assert (spec.num_kv_heads, spec.head_dim, spec.window) == (nkv, hd, window)
    k_pages = torch.full((64, nkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    cache = LayerCache(k_pages, k_pages.clone(), group=0, page_size=page)
    out = attn.forward(ctx, x.to(DEV, dtype), cache, None)

    t = {k: v.double() for k, v in tensors.items()}
    want, off = [], 0
    inv = plain_model.rope_inv_freq(hd, 10000.0, None)
    for n in lens:
        xs = x[off:off + n].double()
        q = xs @ t["q_proj.weight"].T + (t["q_proj.bias"] if bias else 0)
        k = xs @ t["k_proj.weight"].T + (t["k_proj.bias"] if bias else 0)
        v = xs @ t["v_proj.weight"].T + (t["v_proj.bias"] if bias else 0)
        pos = torch.arange(n)
        q = plain_model.apply_rope(q.view(n, nh, hd), pos, inv)
        k = plain_model.apply_rope(k.view(n, nkv, hd), pos, inv)
        a = plain_model.causal_attention(q, k, v.view(n, nkv, hd), 1 / math.sqrt(hd), window)
        want.append(a.reshape(n, nh * hd) @ t["o_proj.weight"].T)
        off += n
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(out.cpu().double(), torch.cat(want), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part_alone(dtype):
    from helios_b200.parts import SwiGLU

    g = torch.Generator().manual_seed(1)
    ffn = SwiGLU(80, 176)
    t = {k: torch.randn(s.shape, generator=g) * 0.1 for k, s in ffn.weight_specs().items()}
    if dtype == torch.bfloat16:
        t = {k: v.to(torch.bfloat16).float() for k, v in t.items()}
    ffn.bind({k: v.to(DEV, dtype) for k, v in t.items()})
    x = torch.randn(19, 80, generator=g).to(dtype)
    want = plain_model.swiglu(x.double(), t["gate_proj.weight"].double(), t["up_proj.weight"].double(),
                              t["down_proj.weight"].double())
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=3e-2)
    torch.testing.assert_close(ffn.forward(None, x.to(DEV)).cpu().double(), want, **tol)


def test_embedding_and_head_parts():
    from helios_b200.parts import OutputHead, TokenEmbedding

    g = torch.Generator().manual_seed(2)
    table = torch.randn(331, 40, generator=g)
    emb, head = TokenEmbedding(331, 40), OutputHead(331, 40)
    emb.bind({"weight": table.to(DEV)})
    head.bind({"weight": table.to(DEV)})
    ctx, _ = _ctx([[5, 330, 0]], torch.float32)
    torch.testing.assert_close(emb.forward(ctx).cpu(), table[[5, 330, 0]])
    rows = torch.randn(4, 40, generator=g)
    torch.testing.assert_close(head.forward(ctx, rows.to(DEV)).cpu().double(), rows.double() @ table.double().T,
                               atol=1e-5, rtol=1e-5)


# ---------------------------------------------------------------------- the schedule is data
@pytest.mark.parametrize("lens", [[20], [1, 1, 1, 1, 1, 1, 1], [9, 1, 12]])
@pytest.mark.parametrize("bias", [False, True])
def test_the_parts_hand_a_norm_to_one_another(lens, bias, monkeypatch):
    """Steps of few tokens in bfloat16: the attention part adds its output into the residual
    and leaves the feed-forward's norm all but done (a DeferredNorm: rows times the norm
    weight, partial sums of squares); the feed-forward takes it, applies 1 / rms inside its
    first product and adds into the residual too.  Against the plain functions."""
    from helios_b200.csrc import ops
    from helios_b200.parts import DeferredNorm, GQAAttention, LayerCache, RMSNorm, RotaryEncoding, SwiGLU

    monkeypatch.setattr(ops, "DEFERRED_NORM_TOKENS", ops.DEFERRED_NORM_MOST)   # also the 32-token tile
    H, I, nh, nkv, hd, page, eps = 2304, 640, 6, 2, 64, 8, 1e-5     # wider than the narrow-model kernels take
    g = torch.Generator().manual_seed(len(lens) + bias)
    attn, ffn = GQAAttention(H, nh, nkv, hd, 1 / math.sqrt(hd), bias), SwiGLU(H, I)
    norm1, norm2 = RMSNorm(H, eps), RMSNorm(H, eps)
    t = {}
    for name, part in (("a.", attn), ("f.", ffn), ("n1.", norm1), ("n2.", norm2)):
        w = {k: (torch.randn(sp.shape, generator=g) * 0.03 if len(sp.shape) == 2
                 else 1.0 + 0.2 * torch.randn(sp.shape, generator=g)) for k, sp in part.weight_specs().items()}
        w = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in w.items()}
        part.bind({k: v.to(DEV, torch.bfloat16 if v.dim() == 2 else torch.float32) for k, v in w.items()})
        t.update({name + k: v.double() for k, v in w.items()})
    ctx, _lay = _ctx([[0] * n for n in lens], torch.bfloat16, page_size=page)
    RotaryEncoding(hd, 10000.0).prepare(ctx)
    T = sum(lens)
    res0 = torch.randn(T, H, generator=g) * 2.0
    residual = res0.to(DEV).clone()
    k_pages = torch.full((64, nkv, page, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    cache = LayerCache(k_pages, k_pages.clone(), group=0, page_size=page)

    handed = attn.forward_from_residual(ctx, residual, norm1, cache, None, pre=None, then=norm2)
    assert isinstance(handed, DeferredNorm) and handed.norm is norm2
    inv = plain_model.rope_inv_freq(hd, 10000.0, None)
    want, off = [], 0
    for n in lens:
        xs = plain_model.rms_norm(res0[off:off + n].double(), t["n1.weight"], eps)
        q = xs @ t["a.q_proj.weight"].T + (t["a.q_proj.bias"] if bias else 0)
        k = xs @ t["a.k_proj.weight"].T + (t["a.k_proj.bias"] if bias else 0)
        v = xs @ t["a.v_proj.weight"].T + (t["a.v_proj.bias"] if bias else 0)
        pos = torch.arange(n)
        a = plain_model.causal_attention(plain_model.apply_rope(q.view(n, nh, hd), pos, inv),
                                         plain_model.apply_rope(k.view(n, nkv, hd), pos, inv),
                                         v.view(n, nkv, hd), 1 / math.sqrt(hd), None)
        want.append(res0[off:off + n].double() + a.reshape(n, nh * hd) @ t["a.o_proj.weight"].T)
        off += n
    after_attn = torch.cat(want)
    torch.testing.assert_close(residual.cpu().double(), after_attn, atol=3e-2, rtol=3e-2)
    got = residual.cpu()
    assert torch.equal(handed.scaled.cpu(), (got * t["n2.weight"].float()).to(torch.bfloat16))
    torch.testing.assert_close(handed.sumsq.cpu().double().sum(1), (got.double() ** 2).sum(1), rtol=1e-5, atol=0)

    assert ffn.forward_from_residual(ctx, residual, norm2, pre=handed, then=None) is True
    xs = plain_model.rms_norm(got.double(), t["n2.weight"], eps)
    want = got.double() + plain_model.swiglu(xs, t["f.gate_proj.weight"], t["f.up_proj.weight"],
                                             t["f.down_proj.weight"])
    torch.testing.assert_close(residual.cpu().double(), want, atol=3e-2, rtol=3e-2)
    # without anything handed over the feed-forward norms by itself, to the same result
    again = got.to(DEV).clone()
    assert ffn.forward_from_residual(ctx, again, norm2, pre=None, then=None) is True
    torch.testing.assert_close(again.cpu().double(), want, atol=3e-2, rtol=3e-2)
    # a norm of another kind next: nothing is prepared for it
    assert attn.forward_from_residual(ctx, res0.to(DEV).clone(), norm1, cache, None, pre=None, then=object()) is True


def _toy_plan(schedule, layers=2):
    from helios_b200.config import DenseDecoderConfig
    from helios_b200.models import build_dense_decoder_plan
    from helios_b200.parts import Run

    cfg = DenseDecoderConfig.from_hf(dict(TINY_LLAMA, num_hidden_layers=layers))
    plan = build_dense_decoder_plan(cfg)
    plan.schedule = [Run(*r) if isinstance(r, tuple) else Run(r) for r in schedule]
    plan.__post_init__()
    return cfg, plan


def _run_plan(plan, toks, cut, dtype=torch.float32):
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel
    from helios_b200.weights import bind_random_weights

    bind_random_weights(plan, 3, dtype, DEV)
    core = EngineCore(DecoderModel(plan, dtype, DEV), page_size=8, num_pages=32, max_slots=2,
                      poison_cache=float("nan"), use_cuda_graphs=False)
    outs = []
    for a, b in zip(cut[:-1], cut[1:]):
        outs.append(core.step([StepEntry("r", toks[a:b], list(range(b - a)))]).clone())
    return torch.cat(outs), core


def test_a_layer_named_twice_runs_twice_with_a_cache_for_each_run():
    toks = random_tokens(256, 30, 5)
    cfg, plan = _toy_plan([0, 1, 0])
    whole, core = _run_plan(plan, toks, [0, 30])
    assert len(core.cache._where) == 3                       # three runs, three caches
    # the same weights laid out as a three-layer model give the same logits
    hf = dict(TINY_LLAMA, num_hidden_layers=3)
    tensors = _export(plan)
    for name, t in list(tensors.items()):
        if name.startswith("model.layers.0."):
            tensors[name.replace("layers.0.", "layers.2.")] = t
    want = plain_model.forward_logits(hf, tensors, toks)
    assert_logits_close(whole, want, "float32", "layer named twice")
    # and cutting the sequence changes nothing
    cfg2, plan2 = _toy_plan([0, 1, 0])
    parts, _ = _run_plan(plan2, toks, [0, 7, 9, 30])
    assert_logits_close(parts, want, "float32", "layer named twice, in portions")


def _export(plan):
    """Checkpoint tensors (float32, CPU) back out of the bound parts of a dense plan."""
    cfg = plan.config
    q, kv = cfg.q_size, cfg.kv_size
    out = {"model.embed_tokens.weight": plan.embedding.table.float().cpu(),
           "model.norm.weight": plan.final_norm.weight.float().cpu(),
           "lm_head.weight": plan.head.weight.float().cpu()}
    for i, block in enumerate(plan.layers):
        p = f"model.layers.{i}."
        m, f = block.mixer, block.ffn
        w = m.w_qkv.float().cpu()
        out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"], out[p + "self_attn.v_proj.weight"] = \
            w[:q], w[q:q + kv], w[q + kv:]
        if m.b_qkv is not None:
            b = m.b_qkv.float().cpu()
            out[p + "self_attn.q_proj.bias"], out[p + "self_attn.k_proj.bias"], out[p + "self_attn.v_proj.bias"] = \
                b[:q], b[q:q + kv], b[q + kv:]
        out[p + "self_attn.o_proj.weight"] = m.w_o.float().cpu()
        gu = f.w_gate_up.float().cpu()
        out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = gu[:f.inner], gu[f.inner:]
        out[p + "mlp.down_proj.weight"] = f.w_down.float().cpu()
        out[p + "input_layernorm.weight"] = block.mixer_norm.weight.float().cpu()
        out[p + "post_attention_layernorm.weight"] = block.ffn_norm.weight.float().cpu()
    return out


def test_a_layer_may_read_another_layers_cache():
    """Entry 1 runs layer 1's weights but attends over the keys and values entry 0 wrote
    (its own k and v are computed and dropped).  Whole and in portions must agree, which
    they only do if the shared cache is read correctly across steps."""
    toks = random_tokens(256, 26, 6)
    _, plan = _toy_plan([0, (1, 0, False)])
    whole, core = _run_plan(plan, toks, [0, 26])
    assert len(core.cache._where) == 1 and core.cache.storage[0].shape[0] == 1
    _, plan2 = _toy_plan([0, (1, 0, False)])
    parts, _ = _run_plan(plan2, toks, [0, 3, 4, 20, 26])
    torch.testing.assert_close(parts, whole, atol=2e-5, rtol=0)
    # and it is not the same as two ordinary layers
    _, plain_plan = _toy_plan([0, 1])
    ordinary, _ = _run_plan(plain_plan, toks, [0, 26])
    assert (ordinary - whole).abs().max() > 1e-4
    with pytest.raises(ValueError):
        _toy_plan([0, (1, 0, True)])          # a shared cache must not be written twice
    with pytest.raises(ValueError):
        _toy_plan([(0, 1, False), 1])         # nor read before anyone owns it


# ---------------------------------------------------------------------- a toy mixer with state
def test_a_toy_mixer_with_state_of_its_own_is_registered_built_and_stepped():
    """A running mean over the request's tokens: state of fixed size per request (sum and
    count), no pages.  Defined here, registered under a name, chosen by a toy
    architecture's plan builder for every second layer; whole sequences, portions and a
    batch of two requests must agree, and a slot handed to a new request starts from zero."""
    from helios_b200.config import DenseDecoderConfig, register_architecture, unregister_architecture
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel
    from helios_b200.parts import (Mixer, ModelPlan, OutputHead, StateSpec, TokenEmbedding, WeightSpec,
                                   part_class, register_part)

    class RunningMean(Mixer):
        graph_safe = False                      # it walks the requests on the host

        def __init__(self, width):
            self.width = width

        def state_spec(self):
            return StateSpec((self.width + 1,), torch.float32)     # sum, count

        def weight_specs(self):
            return {"mix.weight": WeightSpec((self.width, self.width))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"]

        def forward(self, ctx, x, cache, state):
            assert cache is None
            out = torch.empty_like(x)
            for seq in ctx.seqs:
                rows = slice(seq.token_offset, seq.token_offset + seq.num_tokens)
                xs = x[rows].float()
                st = state[seq.slot]
                csum = st[: self.width] + xs.cumsum(0)
                cnt = st[self.width] + torch.arange(1, seq.num_tokens + 1, device=x.device)
                out[rows] = ((csum / cnt[:, None]) @ self.w.float().T).to(x.dtype)
                st[: self.width] = csum[-1]
                st[self.width] = cnt[-1]
            return out

    register_part("mixer", "toy_running_mean", RunningMean, replace=True)

    def build(cfg):
        norm, ffn, block = part_class("norm", "rmsnorm"), part_class("feed_forward", "swiglu"), part_class("block", "pre_norm")
        attn, toy = part_class("mixer", "gqa_attention"), part_class("mixer", "toy_running_mean")
        layers = []
        for i in range(cfg.num_hidden_layers):
            mixer = toy(cfg.hidden_size) if i % 2 else attn(cfg.hidden_size, cfg.num_attention_heads,
                                                            cfg.num_key_value_heads, cfg.head_dim,
                                                            cfg.attention_scale, False)
            layers.append(block(norm(cfg.hidden_size, cfg.rms_norm_eps), mixer,
                                norm(cfg.hidden_size, cfg.rms_norm_eps), ffn(cfg.hidden_size, cfg.intermediate_size)))
        return ModelPlan(config=cfg, embedding=TokenEmbedding(cfg.vocab_size, cfg.hidden_size),
                         position=part_class("position_encoding", "rotary")(cfg.head_dim, cfg.rope_theta),
                         layers=layers, layer_prefixes=[f"model.layers.{i}." for i in range(cfg.num_hidden_layers)],
                         final_norm=norm(cfg.hidden_size, cfg.rms_norm_eps),
                         head=OutputHead(cfg.vocab_size, cfg.hidden_size))

    register_architecture("ToyMeanForCausalLM", lambda d: DenseDecoderConfig.from_hf(d, "ToyMeanForCausalLM"),
                          build, replace=True)
    try:
        cfg_json = dict(TINY_LLAMA, architectures=["ToyMeanForCausalLM"], num_hidden_layers=3, rope_scaling=None)
        for dtype in ("float32", "bfloat16"):
            model = DecoderModel.from_config(cfg_json, seed=4, dtype=dtype)
            assert not model.plan.graph_safe
            core = EngineCore(model, page_size=8, num_pages=32, max_slots=2)
            assert list(core.cache.states) == [1] and core.cache.states[1].shape == (2, 65)
            assert len(core.cache._where) == 2               # only the attention layers have pages
            a, b = random_tokens(256, 23, 1), random_tokens(256, 9, 2)
            whole_a = core.step([StepEntry("a", a, list(range(23)))]).clone()
            core.end("a")
            whole_b = core.step([StepEntry("b", b, list(range(9)))]).clone()     # reuses a's slot: zeroed
            core.end("b")
            got_a, got_b = [], []
            for (sa, ea), (sb, eb) in zip([(0, 5), (5, 6), (6, 20), (20, 23)], [(0, 2), (2, 3), (3, 8), (8, 9)]):
                out = core.step([StepEntry("a", a[sa:ea], list(range(ea - sa))),
                                 StepEntry("b", b[sb:eb], list(range(eb - sb)))])
                got_a.append(out[: ea - sa].clone())
                got_b.append(out[ea - sa:].clone())
            tol = dict(atol=3e-5, rtol=0) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
            torch.testing.assert_close(torch.cat(got_a), whole_a, **tol)
            torch.testing.assert_close(torch.cat(got_b), whole_b, **tol)
            # the toy layer matters: without the state carried over, portions would differ
            assert (whole_a[5] - whole_a[4]).abs().max() > 0
    finally:
        unregister_architecture("ToyMeanForCausalLM")


# ---------------------------------------------------------------------- a toy feed-forward with routing, another position encoding
def test_a_toy_routed_feed_forward_and_a_learned_position_encoding_are_registered_built_and_stepped():
    """Two more parts defined here, not in the package: a feed-forward that sends every
    token to the one of three small experts its router picks (router logits in float32),
    and a position encoding that adds a learned row per position to the embedded tokens
    (attention then runs without rotation).  A toy architecture uses the routed
    feed-forward in every second layer.  The engine's logits are compared with a plain
    computation on whole sequences written out below, and must not depend on how the
    tokens are cut or batched."""
    from helios_b200.config import DenseDecoderConfig, register_architecture, unregister_architecture
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel
    from helios_b200.parts import (FeedForward, ModelPlan, OutputHead, PositionEncoding, TokenEmbedding,
                                   WeightSpec, part_class, register_part)

    E, INNER, MAX_POS = 3, 40, 64

    class RoutedFeedForward(FeedForward):
        graph_safe = False                      # the tokens of an expert are gathered on the host's say

        def __init__(self, width):
            self.width = width

        def weight_specs(self):
            specs = {"router.weight": WeightSpec((E, self.width), std=0.3)}
            for e in range(E):
                specs[f"experts.{e}.up.weight"] = WeightSpec((INNER, self.width), std=0.3)
                specs[f"experts.{e}.down.weight"] = WeightSpec((self.width, INNER), std=0.3)
            return specs

        def bind(self, tensors):
            self.t = tensors

        def forward(self, ctx, x):
            choice = (x.float() @ self.t["router.weight"].float().T).argmax(-1)
            out = torch.zeros_like(x)
            for e in range(E):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(x[rows].float() @ self.t[f"experts.{e}.up.weight"].float().T)
                    out[rows] = (h @ self.t[f"experts.{e}.down.weight"].float().T).to(x.dtype)
            return out

    class LearnedPositions(PositionEncoding):
        def __init__(self, width):
            self.width = width

        def weight_specs(self):
            return {"weight": WeightSpec((MAX_POS, self.width), std=0.5)}

        def bind(self, tensors):
            self.table = tensors["weight"]

        def embed(self, ctx, hidden):
            return hidden + self.table.float().index_select(0, ctx.positions.long())

    register_part("feed_forward", "toy_routed", RoutedFeedForward, replace=True)
    register_part("position_encoding", "toy_learned", LearnedPositions, replace=True)

    def build(cfg):
        norm, block = part_class("norm", "rmsnorm"), part_class("block", "pre_norm")
        attn, dense, routed = (part_class("mixer", "gqa_attention"), part_class("feed_forward", "swiglu"),
                               part_class("feed_forward", "toy_routed"))
        layers = [block(norm(cfg.hidden_size, cfg.rms_norm_eps),
                        attn(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                             cfg.attention_scale, False, rotary=False),
                        norm(cfg.hidden_size, cfg.rms_norm_eps),
                        routed(cfg.hidden_size) if i % 2 else dense(cfg.hidden_size, cfg.intermediate_size))
                  for i in range(cfg.num_hidden_layers)]
        return ModelPlan(config=cfg, embedding=TokenEmbedding(cfg.vocab_size, cfg.hidden_size),
                         position=part_class("position_encoding", "toy_learned")(cfg.hidden_size),
                         layers=layers, layer_prefixes=[f"model.layers.{i}." for i in range(cfg.num_hidden_layers)],
                         final_norm=norm(cfg.hidden_size, cfg.rms_norm_eps),
                         head=OutputHead(cfg.vocab_size, cfg.hidden_size))

    experts_used = set()

    def plain(cfg, plan, toks):
        """float64, whole sequence, from the tensors the parts were given."""
        f = lambda t: t.double().cpu()
        n = len(toks)
        h = f(plan.embedding.table)[toks] + f(plan.position.table)[:n]
        nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        for block in plan.layers:
            x = plain_model.rms_norm(h, f(block.mixer_norm.weight), cfg.rms_norm_eps)
            qkv = x @ f(block.mixer.w_qkv).T
            q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
            a = plain_model.causal_attention(q.reshape(n, nh, hd), k.reshape(n, nkv, hd), v.reshape(n, nkv, hd),
                                             cfg.attention_scale, None)
            h = h + a.reshape(n, nh * hd) @ f(block.mixer.w_o).T
            x = plain_model.rms_norm(h, f(block.ffn_norm.weight), cfg.rms_norm_eps)
            if isinstance(block.ffn, RoutedFeedForward):
                t = {k_: f(v_) for k_, v_ in block.ffn.t.items()}
                choice = (x @ t["router.weight"].T).argmax(-1)
                experts_used.update(choice.tolist())
                y = torch.zeros_like(x)
                for i in range(n):
                    e = int(choice[i])
                    y[i] = torch.relu(x[i] @ t[f"experts.{e}.up.weight"].T) @ t[f"experts.{e}.down.weight"].T
                h = h + y
            else:
                gu = f(block.ffn.w_gate_up)
                h = h + plain_model.swiglu(x, gu[: block.ffn.inner], gu[block.ffn.inner:], f(block.ffn.w_down))
        x = plain_model.rms_norm(h, f(plan.final_norm.weight), cfg.rms_norm_eps)
        return x @ f(plan.head.weight).T

    register_architecture("ToyRoutedForCausalLM", lambda d: DenseDecoderConfig.from_hf(d, "ToyRoutedForCausalLM"),
                          build, replace=True)
    try:
        cfg_json = dict(TINY_LLAMA, architectures=["ToyRoutedForCausalLM"], num_hidden_layers=4, rope_scaling=None)
        model = DecoderModel.from_config(cfg_json, seed=11, dtype="float32")
        assert not model.plan.graph_safe
        assert any(name.startswith("model.position.") for name in
                   __import__("helios_b200.weights", fromlist=["expected_tensors"]).expected_tensors(model.plan))
        core = EngineCore(model, page_size=8, num_pages=32, max_slots=2)
        a, b = random_tokens(256, 29, 3), random_tokens(256, 12, 4)
        whole_a = core.step([StepEntry("a", a, list(range(29)))]).clone()
        core.end("a")
        want_a = plain(model.config, model.plan, a)
        assert_logits_close(whole_a, want_a, "float32", "toy routed model, whole")
        assert experts_used == set(range(E))       # else the test shows nothing of the routing
        got_a, got_b = [], []
        for (sa, ea), (sb, eb) in zip([(0, 7), (7, 8), (8, 27), (27, 29)], [(0, 2), (2, 5), (5, 11), (11, 12)]):
            out = core.step([StepEntry("a", a[sa:ea], list(range(ea - sa))),
                             StepEntry("b", b[sb:eb], list(range(eb - sb)))])
            got_a.append(out[: ea - sa].clone())
            got_b.append(out[ea - sa:].clone())
        assert_logits_close(torch.cat(got_a), want_a, "float32", "toy routed model, in portions beside another")
        assert_logits_close(torch.cat(got_b), plain(model.config, model.plan, b), "float32", "toy routed model, b")
    finally:
        unregister_architecture("ToyRoutedForCausalLM")


# ---------------------------------------------------------------------- other stages, two encodings, a feed-forward with state
def test_a_toy_plan_with_stages_of_its_own_two_rotary_bases_and_a_feed_forward_with_state():
    """What an architecture may differ in without a change to the engine, all defined here: an
    input stage that scales the embedded tokens, an output stage without a final norm that caps
    the logits, attention layers that rotate by two different bases (local and global layers,
    each handed its own encoding), and a feed-forward that keeps a fixed-size state per request
    (the number of tokens it has seen, which it scales its output by).  Compared with a plain
    computation on whole sequences; portions and a batch of two must agree with it."""
    from helios_b200.config import DenseDecoderConfig, register_architecture, unregister_architecture
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel
    from helios_b200.parts import (FeedForward, ModelPlan, OutputHead, OutputStage, StateSpec, TokenEmbedding,
                                   part_class)

    CAP, THETAS = 3.0, (10000.0, 37.0)

    class ScaledEmbedding(TokenEmbedding):
        def forward(self, ctx):
            return super().forward(ctx) * math.sqrt(self.width)

    class CappedHead(OutputStage):
        """No final norm: the pending add, then logits = CAP * tanh(x W^T / CAP)."""

        def __init__(self, vocab, width):
            self.head = OutputHead(vocab, width)

        def named_parts(self):
            return [("lm_head.", self.head)]

        def forward(self, ctx, residual, delta):
            rows = ctx.want_rows.long()
            x = residual.index_select(0, rows) + delta.index_select(0, rows).float()
            return CAP * torch.tanh(self.head.forward(ctx, x.to(ctx.act_dtype)) / CAP)

    class CountingFeedForward(FeedForward):
        """SwiGLU whose output is divided by (1 + tokens of the request seen so far / 8)."""
        graph_safe = False

        def __init__(self, width, inner):
            self.inner_ffn = part_class("feed_forward", "swiglu")(width, inner)

        def state_spec(self):
            return StateSpec((1,), torch.float32)

        def weight_specs(self):
            return self.inner_ffn.weight_specs()

        def bind(self, tensors):
            self.inner_ffn.bind(tensors)

        def forward(self, ctx, x):
            y = self.inner_ffn.forward(ctx, x).float()
            seen = ctx.part_state(self)
            for seq in ctx.seqs:
                rows = slice(seq.token_offset, seq.token_offset + seq.num_tokens)
                count = seen[seq.slot, 0] + torch.arange(seq.num_tokens, device=x.device)
                y[rows] /= (1 + count / 8)[:, None]
                seen[seq.slot, 0] += seq.num_tokens
            return y.to(x.dtype)

    def build(cfg):
        norm, block = part_class("norm", "rmsnorm"), part_class("block", "pre_norm")
        attn, rope = part_class("mixer", "gqa_attention"), part_class("position_encoding", "rotary")
        ropes = [rope(cfg.head_dim, t) for t in THETAS]
        layers = [block(norm(cfg.hidden_size, cfg.rms_norm_eps),
                        attn(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                             cfg.attention_scale, False, position=ropes[i % 2]),
                        norm(cfg.hidden_size, cfg.rms_norm_eps),
                        CountingFeedForward(cfg.hidden_size, cfg.intermediate_size))
                  for i in range(cfg.num_hidden_layers)]
        return ModelPlan(config=cfg, embedding=ScaledEmbedding(cfg.vocab_size, cfg.hidden_size), position=None,
                         layers=layers, layer_prefixes=[f"model.layers.{i}." for i in range(cfg.num_hidden_layers)],
                         output=CappedHead(cfg.vocab_size, cfg.hidden_size))

    def plain(cfg, plan, toks):
        f = lambda t: t.double().cpu()
        n = len(toks)
        h = f(plan.embedding.table)[toks] * math.sqrt(cfg.hidden_size)
        nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        pos = torch.arange(n)
        for i, block in enumerate(plan.layers):
            inv = plain_model.rope_inv_freq(hd, THETAS[i % 2], None)
            x = plain_model.rms_norm(h, f(block.mixer_norm.weight), cfg.rms_norm_eps)
            q, k, v = (x @ f(block.mixer.w_qkv).T).split([nh * hd, nkv * hd, nkv * hd], dim=-1)
            q = plain_model.apply_rope(q.reshape(n, nh, hd), pos, inv)
            k = plain_model.apply_rope(k.reshape(n, nkv, hd), pos, inv)
            a = plain_model.causal_attention(q, k, v.reshape(n, nkv, hd), cfg.attention_scale, None)
            h = h + a.reshape(n, nh * hd) @ f(block.mixer.w_o).T
            x = plain_model.rms_norm(h, f(block.ffn_norm.weight), cfg.rms_norm_eps)
            gu, inner = f(block.ffn.inner_ffn.w_gate_up), block.ffn.inner_ffn.inner
            y = plain_model.swiglu(x, gu[:inner], gu[inner:], f(block.ffn.inner_ffn.w_down))
            h = h + y / (1 + pos.double() / 8)[:, None]
        return CAP * torch.tanh(h @ f(plan.output.head.weight).T / CAP)

    name = "ToyStagesForCausalLM"
    register_architecture(name, lambda d: DenseDecoderConfig.from_hf(d, name), build, replace=True)
    try:
        cfg_json = dict(TINY_LLAMA, architectures=[name], num_hidden_layers=4, rope_scaling=None)
        model = DecoderModel.from_config(cfg_json, seed=21, dtype="float32")
        from helios_b200.weights import expected_tensors
        assert "model.norm.weight" not in expected_tensors(model.plan)          # no final norm to load
        core = EngineCore(model, page_size=8, num_pages=32, max_slots=2)
        assert sorted(core.cache.other_states) == [0, 1, 2, 3]                  # one counter per layer
        a, b = random_tokens(256, 31, 5), random_tokens(256, 10, 6)
        want_a, want_b = plain(model.config, model.plan, a), plain(model.config, model.plan, b)
        whole = core.step([StepEntry("a", a, list(range(31)))]).clone()
        core.end("a")
        assert_logits_close(whole, want_a, "float32", "toy stages, whole")
        # with one base for every layer the logits would differ: the second encoding is used
        inv0, inv1 = (plain_model.rope_inv_freq(16, t, None) for t in THETAS)
        assert (inv0 - inv1).abs().max() > 0.1
        got_a, got_b = [], []
        for (sa, ea), (sb, eb) in zip([(0, 9), (9, 10), (10, 29), (29, 31)], [(0, 3), (3, 4), (4, 9), (9, 10)]):
            out = core.step([StepEntry("b", b[sb:eb], list(range(eb - sb))),      # b takes a's old slot: zeroed
                             StepEntry("a", a[sa:ea], list(range(ea - sa)))])
            got_b.append(out[: eb - sb].clone())
            got_a.append(out[eb - sb:].clone())
        assert_logits_close(torch.cat(got_a), want_a, "float32", "toy stages, a in portions beside b")
        assert_logits_close(torch.cat(got_b), want_b, "float32", "toy stages, b in portions beside a")
    finally:
        unregister_architecture(name)
