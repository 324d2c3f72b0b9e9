"""Command line in the manner of ``python -m helios.cli``
(python/helios/cli.py:210-306), with its names and meanings of options:

    python -m helios_b200.cli generate --model DIR --prompt "..." [--prompt-ids 1,2,3]
    python -m helios_b200.cli info --model DIR
    python -m helios_b200.cli make-toy-model --out DIR
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def cmd_generate(args: argparse.Namespace) -> int:
    from .config.engine_config import EngineConfig
    from .engine.llm import LLMEngine
    from .engine.types import SamplingParams

    if not args.prompt and not args.prompt_ids:
        raise ValueError("give --prompt or --prompt-ids")
    engine = LLMEngine(EngineConfig(
        model_dir=args.model, kv_cache_bytes=args.kv_mb * 1024 * 1024, block_size=args.block_size,
        max_model_len=args.max_model_len, dtype=args.dtype, max_num_seqs=args.max_seqs,
        max_num_batched_tokens=args.max_batched_tokens, device=args.device,
        enable_chunked_prefill=not args.no_chunked_prefill))
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature,
                            top_p=args.top_p, top_k=args.top_k, seed=args.seed,
                            stop_token_ids=engine.eos_token_ids)
    prompts = list(args.prompt or [])
    for ids in args.prompt_ids or []:
        prompts.append([int(t) for t in ids.split(",") if t.strip()])
    for out in engine.generate(prompts, params):
        print(f"--- {out.request_id} ---")
        print(out.text or f"(token ids: {out.token_ids})")
        reason = out.finish_reason.value if out.finish_reason else "none"
        print(f"[{out.completion_tokens} tokens, finish={reason}]")
    return 0


def cmd_info(args: argparse.Namespace) -> int:
    """Sizes of the model and what a cache budget pays for (python/helios/cli.py:182-207)."""
    from .config.model_config import read_config_json
    from .config.registry import resolve_architecture
    from .parts import PagedCacheSpec

    cfg_json = read_config_json(Path(args.model))
    arch = resolve_architecture(cfg_json)
    cfg = arch.parse_config(cfg_json)
    plan = arch.build_plan(cfg)
    dtype_bytes = 4 if args.dtype == "float32" else 2
    per_page = 0
    groups = {}
    for entry, run in enumerate(plan.schedule):
        mixer = plan.layers[run.layer].mixer
        spec = mixer.cache_spec() if mixer is not None and plan.cache_id(entry) == entry else None
        if isinstance(spec, PagedCacheSpec):
            per_page += 2 * args.block_size * spec.num_kv_heads * spec.head_dim * dtype_bytes
            groups[spec] = groups.get(spec, 0) + 1
    budget = args.kv_mb * 1024 * 1024
    pages = budget // max(1, per_page)
    print(f"model: {args.model} ({arch.name})")
    print(f"  layers={cfg.num_hidden_layers} hidden={cfg.hidden_size} intermediate={cfg.intermediate_size}")
    print(f"  q_heads={cfg.num_attention_heads} kv_heads={cfg.num_key_value_heads}"
          f" head_dim={cfg.head_dim} (GQA group={cfg.group_size})")
    print(f"  vocab={cfg.vocab_size} max_pos={cfg.max_position_embeddings}"
          f" parameters={cfg.num_parameters():,}")
    for spec, n in groups.items():
        kind = "all keys" if spec.window is None else f"window {spec.window}"
        print(f"  cache group: {n} layers, {spec.num_kv_heads} kv heads x {spec.head_dim}, {kind}")
    print(f"KV cache ({args.dtype}, block_size={args.block_size}):")
    print(f"  bytes/block = {per_page:,}")
    print(f"  budget {args.kv_mb} MiB -> {pages:,} blocks -> {pages * args.block_size:,} tokens of KV")
    return 0


def cmd_make_toy_model(args: argparse.Namespace) -> int:
    """A small model folder with random weights (python/helios/cli.py:161-179)."""
    from .weights import write_model_folder

    arch = {"llama": ("LlamaForCausalLM", "llama"), "qwen2": ("Qwen2ForCausalLM", "qwen2")}[args.arch]
    cfg = {
        "architectures": [arch[0]], "model_type": arch[1],
        "vocab_size": args.vocab_size, "hidden_size": args.hidden_size,
        "intermediate_size": args.intermediate_size or 2 * args.hidden_size,
        "num_hidden_layers": args.layers, "num_attention_heads": args.heads,
        "num_key_value_heads": args.kv_heads, "max_position_embeddings": args.max_pos,
        "rms_norm_eps": args.rms_eps, "rope_theta": args.rope_theta,
        "tie_word_embeddings": bool(args.tie), "hidden_act": "silu", "torch_dtype": "float32",
        "attention_bias": args.arch == "qwen2", "bos_token_id": 1, "eos_token_id": 2,
    }
    if args.head_dim:
        cfg["head_dim"] = args.head_dim
    if args.rope_scaling:
        f, lo, hi, orig = args.rope_scaling
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": f, "low_freq_factor": lo,
                               "high_freq_factor": hi, "original_max_position_embeddings": int(orig)}
    if args.sliding_window:
        cfg.update(sliding_window=args.sliding_window, use_sliding_window=True,
                   max_window_layers=args.max_window_layers)
    path = write_model_folder(args.out, cfg, seed=args.seed)
    print(f"wrote toy model to {path}")
    print("  NOTE: random weights -- the output means nothing, but every engine")
    print("  code path (paging, batching, sampling) is real.")
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="helios_b200", description="helios_b200 inference engine")
    sub = ap.add_subparsers(dest="command", required=True)

    def add_engine_args(p):
        p.add_argument("--model", required=True)
        p.add_argument("--kv-mb", type=int, default=512, help="KV cache budget in MiB")
        p.add_argument("--block-size", type=int, default=16)
        p.add_argument("--max-model-len", type=int, default=None)
        p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")

    p = sub.add_parser("generate", help="offline generation")
    add_engine_args(p)
    p.add_argument("--prompt", nargs="+", default=None)
    p.add_argument("--prompt-ids", nargs="+", default=None,
                   help="prompts as comma-separated token ids (no tokenizer needed)")
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--max-seqs", type=int, default=64)
    p.add_argument("--max-batched-tokens", type=int, default=2048)
    p.add_argument("--no-chunked-prefill", action="store_true")
    p.add_argument("--device", default="cuda:0")
    p.set_defaults(func=cmd_generate)

    p = sub.add_parser("make-toy-model", help="write a small random-weight model")
    p.add_argument("--out", required=True)
    p.add_argument("--arch", choices=["llama", "qwen2"], default="llama")
    p.add_argument("--vocab-size", type=int, default=259)
    p.add_argument("--hidden-size", type=int, default=64)
    p.add_argument("--intermediate-size", type=int, default=None)
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--heads", type=int, default=4)
    p.add_argument("--kv-heads", type=int, default=2)
    p.add_argument("--head-dim", type=int, default=None)
    p.add_argument("--max-pos", type=int, default=1024)
    p.add_argument("--rope-theta", type=float, default=10000.0)
    p.add_argument("--rope-scaling", type=float, nargs=4, default=None,
                   metavar=("FACTOR", "LOW", "HIGH", "ORIGINAL_MAX_POS"))
    p.add_argument("--rms-eps", type=float, default=1e-5)
    p.add_argument("--sliding-window", type=int, default=None)
    p.add_argument("--max-window-layers", type=int, default=0)
    p.add_argument("--tie", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    p.set_defaults(func=cmd_make_toy_model)

    p = sub.add_parser("info", help="report derived KV capacity for a model")
    add_engine_args(p)
    p.set_defaults(func=cmd_info)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        return args.func(args)
    except (ValueError, FileNotFoundError) as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 2
    except KeyboardInterrupt:
        print("\ninterrupted", file=sys.stderr)
        return 130


if __name__ == "__main__":
    sys.exit(main())
