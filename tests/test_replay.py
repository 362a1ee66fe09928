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


from rbitnet_b200.replay import schedule_whole as whole, schedule_tail32 as tail32, schedule_batches as batches


def collect_by_manifest(out_dir):
    """request id -> [len, vocab] logits, put together from the step files as manifest.json describes them."""
    man = json.loads((Path(out_dir) / "manifest.json").read_text())
    V = man["vocab_size"]
    rows = {}
    for name, info in man["files"].items():
        arr = np.fromfile(Path(out_dir) / name, dtype="<f4").reshape(len(info["rows"]), V)
        for i, row in enumerate(info["rows"]):
            rows.setdefault(row["id"], {})[row["position"]] = torch.from_numpy(arr[i].copy())
    out = {}
    for r, by_pos in rows.items():
        assert sorted(by_pos) == list(range(len(by_pos))), f"{r}: positions {sorted(by_pos)}"
        out[r] = torch.stack([by_pos[i] for i in range(len(by_pos))])
    return out, man


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
        by_manifest, man = collect_by_manifest(out)
        for r, t in reqs.items():
            assert_close(got[r], ref.logits(t), "float32", f"{name} {r}")
            assert torch.equal(by_manifest[r], got[r])
        assert man["mode"] == "stdin" and set(man["requests"]) == set(reqs)
    # the program's own schedules: the same step lines, made from a file of requests
    rf = tmp_path / "requests.jsonl"
    rf.write_text("\n".join(json.dumps({"id": r, "tokens": t}) for r, t in reqs.items()) + "\n")
    for mode, extra in (("whole", []), ("tail32", []), ("batches", ["--batch-size", "3"])):
        out = tmp_path / f"mode_{mode}"
        rc = main(["--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "256",
                   "--mode", mode, "--requests", str(rf)] + extra, stdin=io.StringIO(""), stdout=io.StringIO(),
                  ops=TorchOps(torch.float32))
        assert rc == 0
        got, man = collect_by_manifest(out)
        for r, t in reqs.items():
            assert_close(got[r], ref.logits(t), "float32", f"--mode {mode} {r}")
        if mode == "batches":      # the second batch uses the first one's slots again
            used = [tuple(man["requests"][r]["slots"]) for r in reqs]
            assert len(set(used)) < len(used)


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
    rf = tmp_path / "requests.json"
    rf.write_text(json.dumps(reqs))
    # step lines on standard input (whole requests, and unequal batches), and the program's own modes
    for mode, steps, max_tokens in (("whole", whole(reqs), 256), ("tail32", None, 256),
                                    ("batches", batches(reqs, 3), 3 * 256), ("batches", None, 3 * 256)):
        out = tmp_path / (mode + ("_stdin" if steps is not None else ""))
        cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
               "--out", str(out), "--max-tokens", str(max_tokens)]
        if steps is None:
            cmd += ["--mode", mode, "--requests", str(rf), "--batch-size", "3"]
        p = subprocess.run(cmd, input="" if steps is None else "\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, env=env, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        if steps is not None:
            assert p.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
            got = collect(steps, out, V)
        else:
            got, _ = collect_by_manifest(out)
        for r, t in reqs.items():
            assert_close(got[r], ref.logits(t), dtype, f"{mode} {r}")


def test_request_files_and_schedules(tmp_path):
    """Both request file formats, and the schedules the program makes from them."""
    from rbitnet_b200.replay import read_requests, schedule_whole, schedule_tail32, schedule_batches
    reqs = {"a": [1, 2, 3], "b": list(range(40)), "c": [7]}
    (tmp_path / "lines.jsonl").write_text("\n".join(json.dumps({"id": k, "tokens": v}) for k, v in reqs.items()) + "\n\n")
    (tmp_path / "object.json").write_text(json.dumps(reqs))
    (tmp_path / "empty.jsonl").write_text("")
    assert read_requests(tmp_path / "lines.jsonl") == reqs and read_requests(tmp_path / "object.json") == reqs
    assert read_requests(tmp_path / "empty.jsonl") == {}

    def fed(steps):          # request -> tokens in the order they are fed; ends exactly once, after the last token
        out, ended = {}, []
        for i, st in enumerate(steps):
            assert st["step"] == i
            for e in st["entries"]:
                assert e["id"] not in ended and e["want"] == list(range(len(e["tokens"])))
                out.setdefault(e["id"], []).extend(e["tokens"])
            ended += st["end"]
        assert sorted(ended) == sorted(reqs)
        return out

    assert fed(schedule_whole(reqs)) == reqs
    tail = schedule_tail32(reqs)
    assert fed(tail) == reqs
    assert [len(e["tokens"]) for st in tail for e in st["entries"] if e["id"] == "b"] == [8] + [1] * 32
    for size in (1, 2, 3):
        steps = schedule_batches(reqs, size)
        assert fed(steps) == reqs
        first = steps[0]["entries"]
        assert len(first) == min(size, 3) and all(len(e["tokens"]) >= 1 for e in first)
        # after a batch's first step every entry brings one token, and no request joins a running batch
        batch_ids = {e["id"] for e in first}
        for st in steps[1:]:
            ids = {e["id"] for e in st["entries"]}
            if ids <= batch_ids:
                assert all(len(e["tokens"]) == 1 for e in st["entries"])
            else:
                assert not (ids & batch_ids)
                batch_ids = ids
