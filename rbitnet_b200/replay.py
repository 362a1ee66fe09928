"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it
drives ``Engine`` — the model, step function, cache and kernels that generation
uses.  Steps are read from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the
logits at the wanted places as little-endian float32 [wanted, vocab], in the
order of the entries and of ``want``.  After every step a line ``done <step>``
is printed and flushed.  The reference has nothing comparable; the nearest is
its documented intention to compare first-step logits with another runner
(docs/GOLDEN_TESTS.md:9-15).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np


def main(argv=None, stdin=None, stdout=None, ops=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    args = ap.parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout

    from .engine import Engine, StepEntry
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    kw = {"ops": ops} if ops is not None else {}
    engine = Engine.load_path(args.model, dtype=args.dtype, max_tokens=args.max_tokens, verbose=True, **kw)
    slots = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.new_sequence()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = out_dir / f".{step}.f32.tmp"
                arr.tofile(tmp)
                tmp.replace(out_dir / f"{step}.f32")
        for rid in rec.get("end", []):
            if rid in slots:
                engine.end_sequence(slots.pop(rid))
        print(f"done {step}", file=stdout, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
