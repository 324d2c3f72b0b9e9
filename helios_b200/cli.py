"""Command line in the manner of ``python -m helios.cli``
(python/helios/cli.py:210-306), with its names and meanings of options:

    python -m helios_b200.cli generate --model DIR --prompt "..." [--prompt-ids 1,2,3]
    python -m helios_b200.cli info --model DIR
    python -m helios_b200.cli make-toy-model --out DIR
"""
from __future__ import annotations

import argparse
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
    """What the model folder holds and what a cache budget pays for, read off the model's
    plan: any registered architecture gets this report (python/helios/cli.py:182-207 prints
    the reference's one architecture from its configuration)."""
    from math import prod

    from .cache.manager import bytes_per_page, cache_groups_of, pool_sizes_for_bytes
    from .config.model_config import read_config_json
    from .config.registry import resolve_architecture
    from .weights.loader import expected_tensors

    cfg_json = read_config_json(Path(args.model))
    arch = resolve_architecture(cfg_json)
    plan = arch.build_plan(arch.parse_config(cfg_json))
    stored = {n: spec for n, (_p, _l, spec) in expected_tensors(plan).items() if n not in plan.tied}
    params = sum(prod(spec.shape) for spec in stored.values())
    print(f"{args.model}: {arch.name}")
    print(f"  {len(plan.layers)} layers, {len(plan.schedule)} runs a step; vocabulary {plan.vocab_size:,}; "
          f"{params:,} parameters in {len(stored)} tensors"
          + (f" ({len(plan.tied)} tied to another)" if plan.tied else ""))
    kinds = {}
    for block in plan.layers:
        key = f"{type(block).__name__}(" + ", ".join(type(p).__name__ for _n, p in block.named_parts()) + ")"
        kinds[key] = kinds.get(key, 0) + 1
    for key, n in kinds.items():
        print(f"  {n} x {key}")
    if plan.position is not None:
        print(f"  positions: {type(plan.position).__name__}")
    dtype_bytes = 4 if args.dtype == "float32" else 2
    specs, where = cache_groups_of(plan)
    per_page = bytes_per_page(plan, args.block_size, dtype_bytes)
    budget = args.kv_mb * 1024 * 1024
    pages = pool_sizes_for_bytes(plan, args.block_size, dtype_bytes, budget, args.max_seqs,
                                 args.max_batched_tokens)
    print(f"cache of {args.kv_mb} MiB in {args.dtype}, pages of {args.block_size} tokens, "
          f"{args.max_seqs} request slots:")
    for g, spec in enumerate(specs):
        n_ids = sum(1 for gg, _ in where.values() if gg == g)
        keeps = "every key" if spec.window is None else f"the last {spec.window} keys"
        print(f"  group {g}: {n_ids} caches of {spec.num_kv_heads} KV heads x {spec.head_dim}, keeps {keeps}: "
              f"{per_page[g]:,} bytes a page, {pages[g]:,} pages = {pages[g] * args.block_size:,} tokens")
    full = [n for n, s in zip(pages, specs) if s.window is None]
    if full:
        print(f"  longest context: {min(full) * args.block_size:,} tokens (all requests together)")
    elif specs:
        print("  every cache has a window: the pools bound no request's length")
    return 0


def cmd_make_toy_model(args: argparse.Namespace) -> int:
    """A small model folder with random weights of any registered architecture that offers a
    toy configuration (python/helios/cli.py:161-179)."""
    from .config.registry import find_architecture
    from .weights import write_model_folder

    arch = find_architecture(args.arch)
    if arch.toy_config is None:
        raise ValueError(f"architecture {arch.name} registers no toy configuration")
    sizes = {k: getattr(args, k) for k in (
        "vocab_size", "hidden_size", "intermediate_size", "layers", "heads", "kv_heads", "head_dim",
        "max_pos", "rope_theta", "rope_scaling", "rms_eps", "sliding_window", "max_window_layers", "tie")}
    path = write_model_folder(args.out, arch.toy_config(sizes), seed=args.seed)
    print(f"{arch.name} with random weights (seed {args.seed}) written to {path}")
    print("  its text is noise; pages, batches, portions and sampling work as with any model")
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
    p.add_argument("--arch", default="llama",
                   help="a registered architecture, or the start of its name (llama, qwen2)")
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
    p.add_argument("--max-seqs", type=int, default=64)
    p.add_argument("--max-batched-tokens", type=int, default=2048)
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
