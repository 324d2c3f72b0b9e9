"""Trace replay: feeds given token ids through a model step by step and writes the
logits at the wanted places.  It samples nothing and has no model code of its
own: it drives ``EngineCore.step``, the function generation uses.

Input (standard input, one JSON object a line):

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step with wanted places, ``<out>/<step>.f32`` receives the logits
[wanted, vocab] as little-endian float32, in the order of the entries and of
their ``want``.  After every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=8, help="request slots")
    ap.add_argument("--device", default="cuda:0")
    return ap


def main(argv=None, stdin=None, stdout=None) -> int:
    args = build_parser().parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if args.max_tokens <= 0 or args.block_size <= 0:
        print("error: --max-tokens and --block-size must be positive", file=sys.stderr)
        return 2

    from .batch import StepEntry
    from .core import EngineCore
    from .model import DecoderModel

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = DecoderModel.from_folder(args.model, dtype=args.dtype, device=args.device)
    # Every request's count is rounded up to a multiple of 64 or of the page size,
    # whichever is larger; the pool holds exactly that many tokens in every group.
    unit = max(64, args.block_size)
    unit = -(-unit // args.block_size) * args.block_size
    tokens = -(-args.max_tokens // unit) * unit
    core = EngineCore(model, page_size=args.block_size, num_pages=tokens // args.block_size,
                      max_slots=args.max_live)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in obj.get("entries", [])]
        logits = core.step(entries) if entries else None
        if logits is not None:
            logits.detach().to("cpu").numpy().astype("<f4", copy=False).tofile(str(out_dir / f"{step}.f32"))
        for rid in obj.get("end", []):
            core.end(rid)
        stdout.write(f"done {step}\n")
        stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
