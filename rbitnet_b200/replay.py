"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it
drives ``Engine`` — the model, step function, cache and kernels that generation
uses.  Steps are read from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the
logits at the wanted places as little-endian float32 [wanted, vocab], in the
order of the entries and of ``want``.  After every step a line ``done <step>``
is printed and flushed.

Instead of step lines the program can make the schedule itself from a file of
requests (``--requests FILE``: JSON lines ``{"id": ..., "tokens": [...]}``, or
one JSON object id -> tokens) with ``--mode``:

    whole     each request alone, all its tokens in one step
    tail32    all but the last 32 tokens in one step, then the last 32 one by one
    batches   requests in order in batches of --batch-size; the first half of each
              (--prompt-frac) in one step, then one token each; shorter requests
              end earlier; the next batch uses the slots again

Every logit is asked for in these modes.  In every mode ``<out>/manifest.json``
is written when the input ends: for each step file, which request, position,
slot and row each of its logits rows belongs to.  The reference has nothing
comparable; the nearest is its documented intention to compare first-step
logits with another runner (docs/GOLDEN_TESTS.md:9-25).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Dict, Iterable, Iterator, List


# ------------------------------------------------------------------ schedules
def schedule_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    return [{"step": i, "entries": [{"id": r, "tokens": list(t), "want": list(range(len(t)))}], "end": [r]}
            for i, (r, t) in enumerate(reqs.items())]


def schedule_tail32(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    steps, n = [], 0
    for r, t in reqs.items():
        k = max(1, len(t) - tail)
        steps.append({"step": n, "entries": [{"id": r, "tokens": list(t[:k]), "want": list(range(k))}],
                      "end": [r] if k == len(t) else []})
        n += 1
        for j in range(k, len(t)):
            steps.append({"step": n, "entries": [{"id": r, "tokens": [t[j]], "want": [0]}],
                          "end": [r] if j == len(t) - 1 else []})
            n += 1
    return steps


def schedule_batches(reqs: Dict[str, List[int]], size: int, prompt_frac: float = 0.5) -> List[dict]:
    steps, n = [], 0
    ids = list(reqs)
    for b in range(0, len(ids), size):
        grp = ids[b:b + size]
        plen = {r: max(1, int(len(reqs[r]) * prompt_frac)) for r in grp}
        ends = [r for r in grp if plen[r] == len(reqs[r])]
        steps.append({"step": n, "entries": [{"id": r, "tokens": list(reqs[r][:plen[r]]),
                                              "want": list(range(plen[r]))} for r in grp], "end": ends})
        n += 1
        k = 0
        live = [r for r in grp if r not in ends]
        while live:
            ends = [r for r in live if plen[r] + k + 1 == len(reqs[r])]
            steps.append({"step": n, "entries": [{"id": r, "tokens": [reqs[r][plen[r] + k]], "want": [0]}
                                                 for r in live], "end": ends})
            n += 1
            k += 1
            live = [r for r in live if r not in ends]
    return steps


def read_requests(path) -> Dict[str, List[int]]:
    text = Path(path).read_text().strip()
    if not text:
        return {}
    try:
        whole = json.loads(text)
        if isinstance(whole, dict) and "tokens" not in whole:
            return {str(k): [int(x) for x in v] for k, v in whole.items()}
    except json.JSONDecodeError:
        pass
    out: Dict[str, List[int]] = {}
    for line in text.splitlines():
        if line.strip():
            rec = json.loads(line)
            out[str(rec["id"])] = [int(x) for x in rec["tokens"]]
    return out


def _steps_from(stdin) -> Iterator[dict]:
    for line in stdin:
        line = line.strip()
        if line:
            yield json.loads(line)


# ------------------------------------------------------------------ the program
def run_steps(engine, steps: Iterable[dict], out_dir: Path, stdout) -> dict:
    """Runs the steps on the engine, writes the step files and returns the manifest."""
    from .engine import StepEntry
    slots, fed = {}, {}
    manifest = {"vocab_size": int(engine.model.vocab_size), "files": {}, "requests": {}}
    for rec in steps:
        step = rec["step"]
        entries, rows = [], []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.new_sequence()
                fed[rid] = 0
                manifest["requests"].setdefault(str(rid), {"slots": []})["slots"].append(slots[rid])
            want = list(e.get("want", []))
            entries.append(StepEntry(slots[rid], e["tokens"], want))
            rows += [{"id": rid, "position": fed[rid] + w, "slot": slots[rid]} for w in want]
            fed[rid] += len(e["tokens"])
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = out_dir / f".{step}.f32.tmp"
                arr.tofile(tmp)
                tmp.replace(out_dir / f"{step}.f32")
                manifest["files"][f"{step}.f32"] = {"step": step, "rows": rows}
        for rid in rec.get("end", []):
            if rid in slots:
                engine.end_sequence(slots.pop(rid))
                fed.pop(rid)
        print(f"done {step}", file=stdout, flush=True)
    return manifest


def main(argv=None, stdin=None, stdout=None, ops=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 and manifest.json")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    ap.add_argument("--mode", choices=["stdin", "whole", "tail32", "batches"], default="stdin",
                    help="stdin: step lines from standard input; else a schedule made from --requests")
    ap.add_argument("--requests", help="file of requests for the schedule modes")
    ap.add_argument("--batch-size", type=int, default=4, help="requests per batch in mode batches")
    ap.add_argument("--prompt-frac", type=float, default=0.5,
                    help="mode batches: share of a request that is its prompt (the rest goes one by one)")
    args = ap.parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if args.mode == "stdin":
        steps: Iterable[dict] = _steps_from(stdin)
    else:
        if not args.requests:
            ap.error(f"--mode {args.mode} needs --requests FILE")
        reqs = read_requests(args.requests)
        steps = {"whole": lambda: schedule_whole(reqs), "tail32": lambda: schedule_tail32(reqs),
                 "batches": lambda: schedule_batches(reqs, args.batch_size, args.prompt_frac)}[args.mode]()

    from .engine import Engine
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    kw = {"ops": ops} if ops is not None else {}
    engine = Engine.load_path(args.model, dtype=args.dtype, max_tokens=args.max_tokens, verbose=True, **kw)
    manifest = run_steps(engine, steps, out_dir, stdout)
    manifest.update(mode=args.mode, dtype=args.dtype, model=str(args.model))
    tmp = out_dir / ".manifest.json.tmp"
    tmp.write_text(json.dumps(manifest))
    tmp.replace(out_dir / "manifest.json")
    return 0


if __name__ == "__main__":
    sys.exit(main())
