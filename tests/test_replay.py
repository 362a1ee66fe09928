"""Trace replay.  On the CPU the program's own logic (parsing, request ids, slots, files) runs on
the torch stand-in for the kernels; on the GPU ``bin/trace_run`` is run as a user runs it, the same
requests whole, with the last 32 tokens one by one, and in unequal batches, in both dtypes."""
import io
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import assert_close, make_model_dir, PlainModel
from tiny import TINY_A, TINY_B, prompts

ROOT = Path(__file__).resolve().parent.parent


def whole(reqs):
    return [{"step": i, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]}
            for i, (r, t) in enumerate(reqs.items())]


def tail32(reqs):
    steps, n = [], 0
    for r, t in reqs.items():
        k = max(1, len(t) - 32)
        steps.append({"step": n, "entries": [{"id": r, "tokens": t[:k], "want": list(range(k))}], "end": []})
        n += 1
        for j in range(k, len(t)):
            steps.append({"step": n, "entries": [{"id": r, "tokens": [t[j]], "want": [0]}],
                          "end": [r] if j == len(t) - 1 else []})
            n += 1
        if k == len(t):
            steps[-1]["end"] = [r]
    return steps


def batches(reqs, size, prompt_frac=0.5):
    steps, n = [], 0
    ids = list(reqs)
    for b in range(0, len(ids), size):
        grp = ids[b:b + size]
        plen = {r: max(1, int(len(reqs[r]) * prompt_frac)) for r in grp}
        ends = [r for r in grp if plen[r] == len(reqs[r])]
        steps.append({"step": n, "entries": [{"id": r, "tokens": reqs[r][:plen[r]], "want": list(range(plen[r]))}
                                             for r in grp], "end": ends})
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


def collect(steps, out_dir, vocab):
    """request id -> [len, vocab] logits, put together from the step files."""
    rows = {}
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        f = Path(out_dir) / f"{st['step']}.f32"
        if not wanted:
            assert not f.exists()
            continue
        arr = np.fromfile(f, dtype="<f4").reshape(wanted, vocab)
        off = 0
        for e in st["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(torch.from_numpy(arr[off].copy()))
                off += 1
    return {r: torch.stack(v) for r, v in rows.items()}


def _requests(vocab, lens, seed):
    return {f"r{i}": p for i, p in enumerate(prompts(lens, vocab, seed))}


def test_replay_logic_on_the_cpu_stand_in(tmp_path):
    from torch_ops import TorchOps
    from rbitnet_b200.replay import main
    folder = make_model_dir(tmp_path / "m", TINY_A, 0)
    ref = PlainModel(folder)
    reqs = _requests(256, [5, 40, 3, 70, 12], 1)
    for name, steps in (("whole", whole(reqs)), ("tail", tail32(reqs)), ("batches", batches(reqs, 3))):
        steps.append({"step": len(steps), "entries": [], "end": []})      # an empty step is legal
        out = tmp_path / name
        stdout = io.StringIO()
        rc = main(["--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "256"],
                  stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=stdout,
                  ops=TorchOps(torch.float32))
        assert rc == 0
        assert stdout.getvalue().split("\n")[:-1] == [f"done {s['step']}" for s in steps]
        got = collect(steps, out, 256)
        for r, t in reqs.items():
            assert_close(got[r], ref.logits(t), "float32", f"{name} {r}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_program(tmp_path, name, dtype):
    cfg, seed = {"A": (TINY_A, 0), "B": (TINY_B, 2)}[name]
    folder = make_model_dir(tmp_path / "m", cfg, seed, store=dtype)
    ref = PlainModel(folder)
    V = cfg["vocab_size"]
    top = cfg["max_position_embeddings"]
    reqs = _requests(V, [33, 5, top, 64, 1, 47, 90], 3)
    env = dict(os.environ, PYTHONPATH="")
    for mode, steps, max_tokens in (("whole", whole(reqs), 256), ("tail", tail32(reqs), 256),
                                    ("batches", batches(reqs, 3), 3 * 256)):
        out = tmp_path / mode
        p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", str(max_tokens)],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                           env=env, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert p.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
        got = collect(steps, out, V)
        for r, t in reqs.items():
            assert_close(got[r], ref.logits(t), dtype, f"{mode} {r}")
