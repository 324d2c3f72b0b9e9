#!/usr/bin/env python3
"""Decode and prefill throughput of helios_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model llama8b|qwen7b|qwen0.5b] [--workload decode|mixed]

Default run: the layer sizes of Llama-3.1-8B with random bfloat16 weights, a decode
batch of 8 at a context of 4,096 tokens; it prints ONE JSON line.  ``value`` is
decoded tokens a second of the step function alone (device-timed), ``e2e`` the same
through the Python entry point (host token ids in, sampled ids out), ``prefill`` a
2,048-token prompt, ``points`` decoding at batch 1 and 64, ``roofline`` the bytes the
decode step has to read over its time.  ``points`` also carries the other two size sets
(``--extra-models``): Qwen2.5-7B sizes (decode, prefill, and the mixed workload of 32
requests with prompts of 128 to 4,096 tokens under a budget of 2,048 tokens a step) and
Qwen2.5-0.5B sizes (decode at batch 1, 64 and 256 from 512 to 1,024 tokens, prefill).
``--model`` makes one of them the headline instead; ``--workload mixed`` runs the mixed
workload through ``LLMEngine`` and reports wall time, tokens a second, the steps by size
and the pages' high-water mark; ``--micro`` times single kernels as chains in a captured
graph (the tables under ``profiles/``).  Synthetic token ids, uniform from a seed.
A decode measurement fills the requests' contexts (prompt steps), runs 64 untimed decode
steps, then the W warm-up steps, then exactly K timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {}
LLAMA_31_8B = MODELS["llama8b"] = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256,
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "attention_bias": False, "tie_word_embeddings": False, "hidden_act": "silu",
    "torch_dtype": "bfloat16",
}
QWEN25_7B = MODELS["qwen7b"] = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 152064,
    "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
    "max_position_embeddings": 32768, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "attention_bias": True, "tie_word_embeddings": False, "hidden_act": "silu",
    "sliding_window": 131072, "use_sliding_window": False, "torch_dtype": "bfloat16",
}
QWEN25_05B = MODELS["qwen0.5b"] = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 151936,
    "hidden_size": 896, "intermediate_size": 4864, "num_hidden_layers": 24,
    "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64,
    "max_position_embeddings": 32768, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "attention_bias": True, "tie_word_embeddings": True, "hidden_act": "silu",
    "sliding_window": 32768, "use_sliding_window": False, "torch_dtype": "bfloat16",
}
MODEL_NAMES = {"llama8b": "Llama-3.1-8B sizes", "qwen7b": "Qwen2.5-7B sizes",
               "qwen0.5b": "Qwen2.5-0.5B sizes"}
CONTEXT = 4096
PREFILL_TOKENS = 2048
#: untimed decode steps between the prompt fill and the W warm-up steps of a decode measurement
#: (named in ``config``): they take the device out of the power state the fill left it in
SETTLE_STEPS = 64
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0=None, t1=None):
        mhz, max_mhz, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.samples:
            if t0 is not None and not (t0 <= ts <= t1 + 0.2):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                mhz.append(int(parts[0]))
                max_mhz = max(max_mhz, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def step_flops(cfg, layers, tokens, ctx_start):
    """Matrix-product and attention flops of a step of ``tokens`` new tokens per request
    starting at context ``ctx_start`` (one request)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_tok = 2 * ((nh + 2 * nkv) * hd * H + nh * hd * H + 3 * H * I)
    attn = 0
    for i in range(tokens):
        attn += 4 * nh * hd * (ctx_start + i + 1)
    return layers * (per_tok * tokens + attn) + 2 * V * H


def decode_bytes(cfg, layers, batch, ctx, dtype_bytes=2):
    """Bytes a decode step must read: every weight it uses once, and the cache of the
    live requests."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    w = layers * ((nh + 2 * nkv) * hd * H + nh * hd * H + 3 * H * I) * dtype_bytes
    w += V * H * dtype_bytes + batch * H * dtype_bytes       # output head (tied or not: read once), embedding rows
    kv = layers * batch * ctx * 2 * nkv * hd * dtype_bytes
    return w + kv


def metric_name(args):
    """The same words in both arms: the dtype is in ``dtype``, not here."""
    if args.workload == "mixed":
        return (f"mixed continuous batching tokens/s ({MODEL_NAMES[args.model]}, {args.requests} requests, "
                f"prompts {args.min_prompt}-{args.max_prompt}, budget {args.budget}, {args.new_tokens} new tokens)")
    return f"decode tokens/s ({MODEL_NAMES[args.model]}, batch {args.batch}, context {args.context})"


def run_reference(args):
    """The unmodified reference (installed under baseline/_ref) through its own public
    API, ``LLMEngine(EngineConfig(...))`` / ``add_request`` / ``step``, on the same model
    sizes, batch and context.  Only the model folder (random weights in its checkpoint
    layout) is written here; nothing of helios_b200 runs."""
    if args.workload != "decode" or args.micro:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference arm runs the decode workload only (the default run's metric)"}))
        return 0
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "helios")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref is missing (pip install --no-index --no-deps --target baseline/_ref)"}))
        return 0
    sys.path.insert(0, ref)
    try:
        import torch
        from helios.core.types import SamplingParams
        from helios.engine import EngineConfig, LLMEngine
    except Exception as exc:                                    # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {exc!r}"[:200]}))
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        return 0

    full_layers = MODELS[args.model]["num_hidden_layers"]
    layers = args.ref_layers or full_layers
    cfg = dict(MODELS[args.model], num_hidden_layers=layers)
    folder = os.path.join(args.ref_dir, f"helios_ref_{args.model}_L{layers}_s{args.seed}")
    t_setup = time.time()
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        from safetensors.torch import save_file
        os.makedirs(folder, exist_ok=True)
        gen = torch.Generator(device="cuda").manual_seed(args.seed)
        H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
        q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]

        def rnd(*shape):
            return (torch.randn(*shape, generator=gen, device="cuda") * 0.02).half().cpu()

        tensors = {"model.embed_tokens.weight": rnd(V, H),
                   "model.norm.weight": torch.ones(H, dtype=torch.float16)}
        if not cfg["tie_word_embeddings"]:
            tensors["lm_head.weight"] = rnd(V, H)
        for i in range(layers):
            p = f"model.layers.{i}."
            tensors.update({
                p + "self_attn.q_proj.weight": rnd(q, H), p + "self_attn.k_proj.weight": rnd(kv, H),
                p + "self_attn.v_proj.weight": rnd(kv, H), p + "self_attn.o_proj.weight": rnd(H, q),
                p + "mlp.gate_proj.weight": rnd(I, H), p + "mlp.up_proj.weight": rnd(I, H),
                p + "mlp.down_proj.weight": rnd(H, I),
                p + "input_layernorm.weight": torch.ones(H, dtype=torch.float16),
                p + "post_attention_layernorm.weight": torch.ones(H, dtype=torch.float16)})
            if cfg["attention_bias"]:
                tensors.update({p + "self_attn.q_proj.bias": rnd(q), p + "self_attn.k_proj.bias": rnd(kv),
                                p + "self_attn.v_proj.bias": rnd(kv)})
        save_file(tensors, os.path.join(folder, "model.safetensors"))
        del tensors
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(dict(cfg, torch_dtype="float16"), f)
        torch.cuda.empty_cache()

    page = 16
    pool_tokens = args.batch * (args.context + 2 * page) + 8 * page
    kv_bytes = pool_tokens * 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    engine = LLMEngine(EngineConfig(
        model_dir=folder, kv_cache_bytes=kv_bytes, block_size=page, max_num_seqs=args.batch,
        max_num_batched_tokens=PREFILL_TOKENS, max_model_len=args.context + 8, device="cuda",
        watermark=0.0))
    setup_s = time.time() - t_setup
    gen = torch.Generator().manual_seed(args.seed)

    def tokens(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()

    # prefill of one 2,048-token prompt
    prefill = None
    if not args.no_prefill:
        engine.add_request("warm", tokens(PREFILL_TOKENS), SamplingParams(max_tokens=1))
        engine.run_until_complete()
        torch.cuda.synchronize()
        engine.add_request("p", tokens(PREFILL_TOKENS), SamplingParams(max_tokens=1))
        t0 = time.perf_counter()
        engine.run_until_complete()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        prefill = {"value": round(PREFILL_TOKENS / ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                   "ms": round(ms, 3),
                   "frac": round(step_flops(cfg, layers, PREFILL_TOKENS, 0) / (ms * 1e-3)
                                 / (load_peaks()["bf16_tflops"] * 1e12), 4)}

    steps, warmup = args.steps, max(3, args.warmup)
    ctx0 = args.context - steps - warmup - SETTLE_STEPS - 64
    for b in range(args.batch):
        engine.add_request(f"e{b}", tokens(ctx0), SamplingParams(max_tokens=steps + warmup + SETTLE_STEPS + 64))
    guard = 0
    while engine.scheduler.waiting or any(not s.is_prefill_done for s in engine.scheduler.running):
        engine.step()
        guard += 1
        if guard > 10000:
            break
    for _ in range(SETTLE_STEPS + warmup):     # the same untimed decode steps as the other arm
        engine.step()
    sampler = ClockSampler()
    sampler.start()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    w0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        engine.step()
    end.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - w0) / steps
    t1 = time.time()
    sampler.stop()
    ms = start.elapsed_time(end) / steps
    running = len(engine.scheduler.running)
    line = {
        "impl": "reference",
        "metric": metric_name(args),
        "value": round(running / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16 (the reference's own choice on CUDA)",
        "data": "synthetic token ids (uniform, seeded), random weights N(0, 0.02)",
        "config": {"model": MODEL_NAMES[args.model], "layers": layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "live_requests": running,
                   "seq_len": args.context, "page_size": page, "parallelism": "single GPU",
                   "api": "helios.engine.LLMEngine.step", "setup_s": round(setup_s, 1),
                   "settle_steps": SETTLE_STEPS},
        "clocks": sampler.summary(t0, t1), "gpu_launches": 0, "prefill": prefill,
        "e2e": {"value": round(running / wall, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 16 * args.batch, "d2h_bytes_per_step": 8 * args.batch},
    }
    print(json.dumps(line))
    return 0


def mixed_prompts(args, vocab, gen):
    """BASELINE config 4's workload: prompt lengths uniform in [min, max], ids uniform."""
    import torch
    lens = torch.randint(args.min_prompt, args.max_prompt + 1, (args.requests,), generator=gen).tolist()
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lens]


def run_mixed(engine, prompts, new_tokens, sampling_cls):
    """All requests at once through ``LLMEngine``; wall time from the first step to the last,
    the device's busy share of it (CUDA events around every launch), the steps by size and the
    pages' high-water mark."""
    import torch

    launch = engine.executor.launch
    marks, sizes = [], []

    def timed_launch(plan, feed=None):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        handle = launch(plan, feed)
        b.record()
        marks.append((a, b))
        sizes.append(plan.num_tokens)
        return handle

    engine.executor.launch = timed_launch
    for i, p in enumerate(prompts):
        engine.add_request(f"m{i}", p, sampling_cls(max_tokens=new_tokens))
    high = 0
    torch.cuda.synchronize()
    w0 = time.perf_counter()
    while engine.scheduler.has_work:
        engine.step()
        high = max(high, max(pool.num_used for pool in engine.core.cache.pools))
    torch.cuda.synchronize()
    wall = time.perf_counter() - w0
    engine.executor.launch = launch
    busy = sum(a.elapsed_time(b) for a, b in marks) * 1e-3
    classes = {"decode_le_64": 0, "le_512": 0, "513_to_1791": 0, "ge_1792": 0}
    for n in sizes:
        key = "decode_le_64" if n <= 64 else "le_512" if n <= 512 else "513_to_1791" if n < 1792 else "ge_1792"
        classes[key] += 1
    done = engine._completed
    generated = sum(o.completion_tokens for o in done)
    prompt_tokens = sum(len(p) for p in prompts)
    return {"wall_s": round(wall, 3), "tokens": prompt_tokens + generated, "generated": generated,
            "tokens_per_s": round((prompt_tokens + generated) / wall, 1),
            "generated_per_s": round(generated / wall, 1), "steps": len(sizes),
            "device_busy": round(busy / wall, 3), "steps_by_tokens": classes,
            "pages_high_water": high, "pages": engine.core.cache.pools[0].num_pages,
            "preemptions": engine.scheduler.stats.preemptions}


def run_micro(args):
    """Single kernels as they follow one another in a step: a captured graph of ``--micro-launches``
    launches of ONE kernel over rotating copies of its weights (more bytes than L2 holds),
    CUDA events around five replays.  Prints one JSON line per case: microseconds a launch and
    the bytes it must read over that time over the measured copy bandwidth."""
    import torch
    from helios_b200.csrc import ops

    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    peaks = load_peaks()
    cfg = MODELS[args.model]
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    n = args.micro_launches
    torch.manual_seed(args.seed)

    def chain_us(fn):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        if n < 8:                       # a profiler's run: a few plain launches
            for i in range(n):
                fn(i)
            torch.cuda.synchronize()
            return float("nan")
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            graph.capture_begin()
            for i in range(n):
                fn(i)
            graph.capture_end()
        torch.cuda.synchronize()
        graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 5 / n * 1e3

    def report(case, us, nbytes, **more):
        frac = nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"] if us == us else None
        print(json.dumps(dict(micro=args.micro, model=MODEL_NAMES[args.model], case=case, us=round(us, 2),
                              hbm_frac=None if frac is None else round(frac, 3), **more)), flush=True)

    def weights(rows, cols):
        copies = max(2, min(96, int(3e9 // (rows * cols * 2))))
        return [(torch.randn(rows, cols, device=dev) * 0.02).bfloat16() for _ in range(copies)]

    if args.micro == "gemm":
        shapes = {"gate_up": (2 * I, H), "down": (H, I), "qkv": ((nh + 2 * nkv) * hd, H), "o": (H, nh * hd)}
        token_counts = [int(t) for t in args.micro_tokens.split(",")] if args.micro_tokens else (8, 16, 32, 64, 128)
        for name, (rows, cols) in shapes.items():
            if args.micro_case and args.micro_case != name:
                continue
            w = weights(rows, cols)
            for T in token_counts:
                x = torch.randn(T, cols, device=dev).bfloat16()
                if name == "gate_up":
                    us = chain_us(lambda i: ops.linear_swiglu(x, w[i % len(w)]))
                else:
                    us = chain_us(lambda i: ops.linear(x, w[i % len(w)]))
                report(name, us, rows * cols * 2, tokens=T)
                if T <= ops.DEFERRED_NORM_MOST:
                    # the epilogues that replace the norm launches in steps of few tokens
                    if name in ("o", "down"):
                        res, nw = torch.randn(T, rows, device=dev), torch.ones(rows, device=dev)
                        us = chain_us(lambda i: ops.linear_bf16(x, w[i % len(w)], residual=res, norm_weight=nw))
                        report(name + "_into_residual_with_next_norm", us, rows * cols * 2, tokens=T)
                    else:
                        ss = torch.rand(T, 8 * -(-cols // 128), device=dev)
                        us = chain_us(lambda i: ops.linear_bf16(x, w[i % len(w)], glu=name == "gate_up",
                                                                sumsq=ss, eps=1e-5))
                        report(name + "_with_rms_factor", us, rows * cols * 2, tokens=T)
            del w
    elif args.micro == "sampling":
        V = cfg["vocab_size"]
        cases = (("greedy", (0.0, 0, 1.0)), ("temperature", (0.8, 0, 1.0)), ("top_k_50", (0.8, 50, 1.0)),
                 ("top_p_09", (0.8, 0, 0.9)), ("top_k_50_top_p_09", (0.8, 50, 0.9)))
        for R in (1, 8, 64, 256):
            logits = torch.randn(R, V, device=dev) * 3
            seeds = torch.arange(R, dtype=torch.int64, device=dev)
            offsets = torch.zeros(R, dtype=torch.int64, device=dev)
            for name, (temp, k, p) in cases:
                t = torch.full((R,), temp, device=dev)
                kk = torch.full((R,), k, dtype=torch.int32, device=dev)
                pp = torch.full((R,), p, device=dev)
                for kernel, kind in (("one block a row", "one_block"), ("cluster a row", "narrow")):
                    us = chain_us(lambda i: ops.sample(logits, t, kk, pp, seeds, offsets, kind=kind))
                    report(name, us, R * V * 4, rows=R, vocab=V, kernel=kernel)
    else:
        B, ctx, page = args.batch, args.context, 16
        pages = B * (ctx // page)
        k = torch.randn(pages, nkv, page, hd, device=dev).bfloat16()
        v = torch.randn_like(k)
        table = torch.randperm(pages, device=dev).int().reshape(B, ctx // page).contiguous()
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=dev).bfloat16()
        nbytes = B * ctx * nkv * hd * 2 * 2
        for splits in sorted({1, 2, 4, 8, ops.decode_splits(B, nkv, ctx)}):
            us = chain_us(lambda i: ops.attention_decode_bf16(qkv, k, v, table, pos, nh, nkv, hd, page, None,
                                                              hd ** -0.5, splits))
            report("attention_decode", us, nbytes, batch=B, context=ctx, splits=splits,
                   chosen=splits == ops.decode_splits(B, nkv, ctx))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama8b", choices=sorted(MODELS),
                    help="the size set of the headline numbers")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the model has (both numbers are reported); 0 = all")
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--points", default="1,64", help="further decode batch sizes")
    ap.add_argument("--extra-models", default=None,
                    help="size sets whose numbers go into ``points`` beside the headline's "
                         "(default: qwen7b,qwen0.5b for the default headline, none otherwise)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--prefill-start", type=int, default=0,
                    help="tokens of the prompt already in the cache when the timed 2,048-token prefill step runs")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-run-ahead", action="store_true",
                    help="end to end: read every step's tokens before the next step is launched")
    ap.add_argument("--no-graphs", action="store_true",
                    help="run decode steps kernel by kernel (for profilers) instead of as captured graphs")
    ap.add_argument("--ref-layers", type=int, default=0,
                    help="layers of the reference arm's model (its loader builds the model in "
                         "float32 on the host first); 0 = all")
    ap.add_argument("--ref-dir", default="/tmp", help="where the reference arm's model folder is written")
    # the mixed workload (BASELINE config 4)
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=4096)
    ap.add_argument("--budget", type=int, default=2048, help="tokens a step (chunked prefill)")
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--micro", default=None, choices=["gemm", "attention_decode", "sampling"],
                    help="time one kind of kernel as a chain in a captured graph instead of the step "
                         "(sizes of --model; --batch tokens or requests, --context keys)")
    ap.add_argument("--micro-case", default=None, help="--micro gemm: one of gate_up, down, qkv, o")
    ap.add_argument("--micro-tokens", default=None, help="--micro gemm: token counts, e.g. 8,16")
    ap.add_argument("--micro-launches", type=int, default=48,
                    help="launches in the chain; below 8 they run plainly, for a profiler")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.micro:
        return run_micro(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from helios_b200.config import EngineConfig
    from helios_b200.csrc import ops
    from helios_b200.engine.batch import StepEntry
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.llm import LLMEngine
    from helios_b200.engine.model import DecoderModel
    from helios_b200.engine.types import SamplingParams

    peaks = load_peaks()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    page = 16
    gen = torch.Generator().manual_seed(args.seed)

    def make_model(name, layers=0):
        full = MODELS[name]["num_hidden_layers"]
        cfg = dict(MODELS[name], num_hidden_layers=layers or full)
        return cfg, full, DecoderModel.from_config(cfg, seed=args.seed, dtype="bfloat16", device=dev)

    def timed_steps(fn, n):
        """(mean, median) milliseconds of ``n`` calls, each between two CUDA events."""
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        torch.cuda.synchronize()
        marks[0].record()
        for i in range(n):
            fn()
            marks[i + 1].record()
        torch.cuda.synchronize()
        each = [marks[i].elapsed_time(marks[i + 1]) for i in range(n)]
        return marks[0].elapsed_time(marks[n]) / n, statistics.median(each)

    def measure_prefill(core, cfg, start=0):
        vocab, layers = cfg["vocab_size"], cfg["num_hidden_layers"]
        times = []
        # the first runs of the shape go kernel by kernel, one more on the graph's buffers, the
        # next captures the graph (EngineCore.FULL_GRAPH_EAGER_RUNS): the last three are replays
        runs = EngineCore.FULL_GRAPH_EAGER_RUNS + 5
        for i in range(runs):
            # the prompt's first ``start`` tokens go into the cache untimed, in portions
            for p0 in range(0, start, PREFILL_TOKENS):
                n = min(PREFILL_TOKENS, start - p0)
                core.step([StepEntry("p", torch.randint(0, vocab, (n,), generator=gen).tolist(), [])])
            toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
            ms, _ = timed_steps(lambda: core.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])]), 1)
            core.end("p")
            if i >= runs - 3:
                times.append(ms)
        ms = statistics.median(times)
        flops = step_flops(cfg, layers, PREFILL_TOKENS, start)
        out = {"value": round(PREFILL_TOKENS / ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
               "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
        if start:
            out["start"] = start
        return out

    def measure_decode(core, cfg, batch, ctx_end, steps, warmup):
        """``steps`` decode steps of ``batch`` requests that end at context ``ctx_end``."""
        vocab = cfg["vocab_size"]
        ctx0 = ctx_end - steps - warmup - SETTLE_STEPS
        for b in range(batch):
            left = ctx0
            while left > 0:
                n = min(left, PREFILL_TOKENS)
                core.step([StepEntry(f"d{b}", torch.randint(0, vocab, (n,), generator=gen).tolist(), [])])
                left -= n
        last = torch.randint(0, vocab, (batch,), generator=gen).tolist()

        def one():
            core.step([StepEntry(f"d{b}", [last[b]], [0]) for b in range(batch)])

        # the prompt fill above is a burst of tensor-core work that leaves the device under its
        # power cap at lowered SM clocks for some 100 ms; untimed decode steps first, so that the
        # timed ones run in the state of a device that is decoding, as a server's do
        for _ in range(SETTLE_STEPS):
            one()
        torch.cuda.synchronize()
        for _ in range(warmup):
            one()
        before = ops.launch_count
        mean, median = timed_steps(one, steps)
        launches = ops.launch_count - before
        for b in range(batch):
            core.end(f"d{b}")
        mean_ctx = ctx0 + SETTLE_STEPS + warmup + steps // 2
        need = decode_bytes(cfg, cfg["num_hidden_layers"], batch, mean_ctx)
        return {"ms": mean, "ms_median": median, "launches": launches, "mean_ctx": mean_ctx,
                "tokens_per_s": batch / mean * 1e3, "gbs": need / (mean * 1e-3) / 1e9}

    def mixed_engine(model, cfg):
        pool_tokens = sum(min(args.max_prompt, 8192) + args.new_tokens + page for _ in range(args.requests))
        return LLMEngine(EngineConfig(
            model_dir="", dtype="bfloat16", block_size=page, max_num_seqs=args.requests,
            max_num_batched_tokens=args.budget, max_model_len=args.max_prompt + args.new_tokens + 8,
            num_blocks=pool_tokens // page + 8, watermark=0.0, run_ahead=not args.no_run_ahead), model=model)

    def measure_mixed(model, cfg):
        """Once to warm up (kernels compiled, shapes seen, graphs captured), once timed, on a
        fresh engine each (the timed one meets the same shapes with its own graphs: captures
        are part of what a server pays, so they are inside the wall time)."""
        g = torch.Generator().manual_seed(args.seed + 1)
        prompts = mixed_prompts(args, cfg["vocab_size"], g)
        run_mixed(mixed_engine(model, cfg), prompts[:4], 8, SamplingParams)
        torch.cuda.empty_cache()
        return run_mixed(mixed_engine(model, cfg), prompts, args.new_tokens, SamplingParams)

    # ---------------------------------------------------------------- the headline model
    cfg, full_layers, model = make_model(args.model, args.layers)
    layers = cfg["num_hidden_layers"]
    sampler = ClockSampler()
    sampler.start()
    config = {"model": MODEL_NAMES[args.model], "layers": layers, "layers_full": full_layers,
              "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
              "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
              "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
              "global_batch": args.batch, "seq_len": args.context, "page_size": page,
              "parallelism": "single GPU", "l2": "inputs (weights + cache) larger than L2",
              "seed": args.seed, "workload": args.workload, "settle_steps": SETTLE_STEPS}

    if args.workload == "mixed":
        t0 = time.time()
        res = measure_mixed(model, cfg)
        clocks = sampler.summary(t0, time.time())
        sampler.stop()
        config.update(global_batch=args.requests, seq_len=args.max_prompt + args.new_tokens)
        line = {"metric": metric_name(args), "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                "steps": res["steps"], "warmup": args.warmup,
                "ms_per_step": round(res["wall_s"] * 1e3 / max(1, res["steps"]), 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic token ids and prompt lengths (uniform, seeded), random weights N(0, 0.02)",
                "impl": "ours", "config": config, "clocks": clocks, "gpu_launches": ops.launch_count,
                "mixed": res,
                "e2e": {"value": res["tokens_per_s"], "unit": "tokens/s",
                        "h2d_bytes_per_step": "token ids, positions and block tables of the step",
                        "d2h_bytes_per_step": "4 per sampled request"}}
        print(json.dumps(line))
        return 0

    point_batches = [int(b) for b in args.points.split(",") if b.strip()]
    max_batch = max([args.batch] + point_batches)
    core = EngineCore(model, page_size=page, num_pages=max_batch * (args.context // page) + 64,
                      max_slots=max_batch, max_model_len=args.context + 1,
                      use_cuda_graphs=not args.no_graphs)
    prefill = None
    if not args.no_prefill:
        if args.prefill_start + PREFILL_TOKENS > args.context:
            raise SystemExit(f"--prefill-start {args.prefill_start} needs --context >= "
                             f"{args.prefill_start + PREFILL_TOKENS}")
        prefill = measure_prefill(core, cfg, args.prefill_start)

    t0 = time.time()
    head = measure_decode(core, cfg, args.batch, args.context, args.steps, args.warmup)
    t1 = time.time()
    clocks = sampler.summary(t0, t1)
    roofline = {"bound": "hbm", "achieved": round(head["gbs"], 1), "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": round(head["gbs"] / peaks["hbm_gbs"], 4),
                "peak_source": peaks["source"]}
    points = {}
    for b in point_batches:
        r = measure_decode(core, cfg, b, args.context, max(8, args.steps // 2), args.warmup)
        points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
        points[f"decode_b{b}_hbm_frac"] = round(r["gbs"] / peaks["hbm_gbs"], 4)

    # ---------------------------------------------------------------- end to end
    e2e = None
    del core
    torch.cuda.empty_cache()
    def measure_e2e(**sampling):
        """Decoded tokens a second through ``LLMEngine.step`` (host ids in, sampled ids out)."""
        engine = LLMEngine(EngineConfig(
            model_dir="", dtype="bfloat16", block_size=page, max_num_seqs=args.batch,
            max_num_batched_tokens=PREFILL_TOKENS, max_model_len=args.context + 8,
            num_blocks=args.batch * (args.context // page + 2) + 8, watermark=0.0,
            run_ahead=not args.no_run_ahead), model=model)
        ctx0 = args.context - args.steps - args.warmup - SETTLE_STEPS
        # every request must still be decoding when the timed steps end, whenever its prompt
        # was finished: the first ones decode while the others' prompts are still being filled
        head_start = max(64, -(-args.batch * ctx0 // PREFILL_TOKENS) + 8)
        if head_start >= ctx0:
            raise SystemExit(f"--batch {args.batch} at --context {args.context}: the prompts take longer "
                             "to fill than the context leaves room for")
        for b in range(args.batch):
            toks = torch.randint(0, cfg["vocab_size"], (ctx0 - head_start,), generator=gen).tolist()
            engine.add_request(f"e{b}", toks, SamplingParams(
                max_tokens=args.steps + args.warmup + SETTLE_STEPS + head_start, seed=b, **sampling))
        while any(s.num_pending_tokens > 1 for s in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        for _ in range(SETTLE_STEPS):        # as in measure_decode: out of the prompt fill's power state
            engine.step()
        for _ in range(args.warmup):
            engine.step()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(args.steps):
            engine.step()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - w0) / args.steps
        return round(args.batch / wall, 1), engine.steps_ahead

    if not args.no_e2e:
        value, ahead = measure_e2e()
        # the same with every request drawing from its top 50 tokens and 0.9 of the mass
        sampled, _ = measure_e2e(temperature=0.8, top_k=50, top_p=0.9)
        h2d = 4 * (args.batch * 8 + args.batch * (args.context // page + 1)) + args.batch * 28
        e2e = {"value": value, "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch,
               "steps_launched_ahead": ahead, "value_top_k_50_top_p_09": sampled}
    sampler.stop()
    del model
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- the other size sets
    extra = args.extra_models
    if extra is None:
        extra = "qwen7b,qwen0.5b" if (args.model == "llama8b" and args.layers in (0, full_layers)) else ""
    for name in [n for n in extra.split(",") if n.strip() and n != args.model]:
        xcfg, _xfull, xmodel = make_model(name)
        if name == "qwen0.5b":
            # BASELINE config 5: 512-token prompts grown to 1,024, batch 1 / 64 / 256
            batches, ctx_end, steps = (1, 64, 256), 1024, 256
        else:
            batches, ctx_end, steps = (64,), args.context, max(8, args.steps // 2)
        xcore = EngineCore(xmodel, page_size=page, num_pages=max(batches) * (ctx_end // page) + 256,
                           max_slots=max(batches), max_model_len=max(ctx_end, PREFILL_TOKENS) + 1)
        points[f"{name}_prefill_{PREFILL_TOKENS}"] = measure_prefill(xcore, xcfg)["value"]
        for b in batches:
            r = measure_decode(xcore, xcfg, b, ctx_end, steps, args.warmup)
            points[f"{name}_decode_b{b}"] = round(r["tokens_per_s"], 1)
            points[f"{name}_decode_b{b}_hbm_frac"] = round(r["gbs"] / peaks["hbm_gbs"], 4)
        del xcore
        torch.cuda.empty_cache()
        if name == "qwen7b":
            res = measure_mixed(xmodel, xcfg)
            points["qwen7b_mixed_tokens_per_s"] = res["tokens_per_s"]
            points["qwen7b_mixed_wall_s"] = res["wall_s"]
            points["qwen7b_mixed_device_busy"] = res["device_busy"]
        del xmodel
        torch.cuda.empty_cache()

    line = {
        "metric": metric_name(args),
        "value": round(head["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(head["ms"], 4),
        "ms_per_step_median": round(head["ms_median"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids (uniform, seeded), random weights N(0, 0.02)",
        "impl": "ours", "config": config,
        "clocks": clocks, "gpu_launches": head["launches"], "prefill": prefill, "roofline": roofline,
        "points": points, "e2e": e2e,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
