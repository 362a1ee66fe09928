"""The step function's host logic on the torch stand-in for the kernels (no GPU): packing without
padding, wanted places, steps cut into batches of rows, guards."""
import pytest
import torch

from helpers import assert_close, make_model_dir, PlainModel
from tiny import TINY_A, TINY_B, prompts
from torch_ops import TorchOps


def _engine(folder, **kw):
    from rbitnet_b200 import Engine
    return Engine.load_path(folder, dtype="float32", ops=TorchOps(torch.float32), max_tokens=2048, **kw)


@pytest.mark.parametrize("cfg,seed", [(TINY_A, 0), (TINY_B, 2)])
@pytest.mark.parametrize("rows_per_batch", [7, 50, 8192])
def test_steps_cut_into_batches_of_rows_give_the_same_logits(tmp_path, cfg, seed, rows_per_batch):
    from rbitnet_b200 import StepEntry
    folder = make_model_dir(tmp_path / "m", cfg, seed)
    ref = PlainModel(folder)
    eng = _engine(folder, max_batch_tokens=rows_per_batch, page_size=16)
    ps = prompts([23, 1, 40, 9], cfg["vocab_size"], 60)
    wants = [[0, 5, 22], [0], [], [8, 3][::-1]]
    slots = [eng.new_sequence() for _ in ps]
    out = eng.step([StepEntry(s, p, w) for s, p, w in zip(slots, ps, wants)])
    assert out.shape[0] == sum(len(w) for w in wants)
    off = 0
    for p, w in zip(ps, wants):
        if w:
            assert_close(out[off:off + len(w)], ref.logits(p)[w], "float32", "wanted places in order")
        off += len(w)
    assert [eng.cache.length(s) for s in slots] == [len(p) for p in ps]
    # nothing wanted: the step still runs and returns nothing
    assert eng.step([StepEntry(slots[1], [3, 4], [])]) is None
    assert eng.cache.length(slots[1]) == 3


def test_step_guards(tmp_path):
    from rbitnet_b200 import StepEntry
    from rbitnet_b200.cache import CacheFull, ContextOverflow
    folder = make_model_dir(tmp_path / "m", TINY_A, 0)
    eng = _engine(folder)
    s = eng.new_sequence()
    with pytest.raises(ValueError, match="out of range"):
        eng.step([StepEntry(s, [1, 256], [])])
    with pytest.raises(ValueError, match="out of range"):
        eng.step([StepEntry(s, [-1], [])])
    with pytest.raises(ValueError, match="at least one token"):
        eng.step([StepEntry(s, [], [])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([StepEntry(s, [1], []), StepEntry(s, [2], [])])
    with pytest.raises(ValueError, match="wanted place"):
        eng.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(ContextOverflow):
        eng.step([StepEntry(s, [1] * 129, [])])
    assert eng.cache.length(s) == 0                  # a refused step leaves the sequence as it was
    small = _engine(folder, max_seq=64)
    small.cache.book.pools[0]._free = small.cache.book.pools[0]._free[:1]      # one page left
    a, b = small.new_sequence(), small.new_sequence()
    small.step([StepEntry(a, [1] * 16, [])])
    with pytest.raises(CacheFull):
        small.step([StepEntry(b, [1], [])])
    with pytest.raises(ValueError, match="exceeds the model"):
        _engine(folder, max_seq=129)


def test_engine_facade_information(tmp_path):
    folder = make_model_dir(tmp_path / "m", TINY_B, 2)
    eng = _engine(folder)
    assert eng.is_ready() and eng.tensor_count() == 30
    assert eng.tensor_names_preview(2) == ["lm_head.weight", "model.embed_tokens.weight"]
    assert "LlamaForCausalLM" in eng.model_summary() and "layers=3" in eng.model_summary()
    from rbitnet_b200.engine import TokenizerMissing
    with pytest.raises(TokenizerMissing):
        eng.complete("hello", 4, 0.0)


def test_command_line_random_and_inspect(tmp_path, capsys):
    import json
    from rbitnet_b200.cli import main
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_A))
    assert main(["random", "--config", str(cfg), "--out", str(tmp_path / "m"), "--seed", "9", "--dtype", "float32"]) == 0
    assert main(["inspect", str(tmp_path / "m"), "--max-names", "2"]) == 0
    out = capsys.readouterr().out
    assert "LlamaForCausalLM: 2 layers, width 64, vocabulary 256" in out and "tensors fit the model" in out
    # the same seed gives the same folder, another seed another one
    assert main(["random", "--config", str(cfg), "--out", str(tmp_path / "m2"), "--seed", "9", "--dtype", "float32"]) == 0
    assert (tmp_path / "m" / "model.safetensors").read_bytes() == (tmp_path / "m2" / "model.safetensors").read_bytes()


def test_engine_from_env(tmp_path, monkeypatch):
    import json
    from rbitnet_b200 import Engine
    from rbitnet_b200.config import ConfigError
    monkeypatch.delenv("RBITNET_MODEL", raising=False)
    monkeypatch.delenv("RBITNET_TOY", raising=False)
    with pytest.raises(ConfigError, match="model not loaded"):
        Engine.from_env(ops=TorchOps(torch.float32), dtype="float32")
    folder = make_model_dir(tmp_path / "m", TINY_A, 0)
    monkeypatch.setenv("RBITNET_MODEL", str(folder))
    eng = Engine.from_env(ops=TorchOps(torch.float32), dtype="float32", max_tokens=256)
    assert eng.tensor_count() == 20
    monkeypatch.setenv("RBITNET_MODEL", str(tmp_path / ".." / "m"))
    with pytest.raises(ValueError, match=r"'\.\.'"):
        Engine.from_env(ops=TorchOps(torch.float32), dtype="float32")
    monkeypatch.delenv("RBITNET_MODEL")
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_A))
    monkeypatch.setenv("RBITNET_TOY", "1")
    monkeypatch.setenv("RBITNET_TOY_CONFIG", str(cfg))
    monkeypatch.setenv("RBITNET_TOY_SEED", "5")
    a = Engine.from_env(ops=TorchOps(torch.float32), dtype="float32", max_tokens=256)
    res = a.generate([[1, 2, 3]], max_tokens=3, temperature=0.0)
    assert len(res[0].tokens) == 3 and res[0].finish_reason == "length"


def test_command_line_generate_on_the_stand_in(tmp_path, capsys):
    """The generate verb's own logic (prompts from arguments and from a file, stop ids, temperature,
    printed records) with the torch stand-in for the kernels; greedy ids equal the plain model's, and a
    temperature run repeats for the same seed."""
    import json
    import plain_llama as plain
    from rbitnet_b200.cli import main
    folder = make_model_dir(tmp_path / "m", TINY_A, 0)
    pc, pt = plain.load_folder(folder)
    prompts_file = tmp_path / "p.txt"
    prompts_file.write_text("9 8 7 6\n\n1, 2\n")
    common = ["generate", "--model", str(folder), "--dtype", "float32", "--cache-tokens", "256", "--max-tokens", "5"]
    assert main(common + ["--temperature", "0", "--stop-id", "3", "--prompt-ids", "5 17 3", "--prompt-ids", str(prompts_file)],
                ops=TorchOps(torch.float32)) == 0
    recs = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
    assert [r["prompt_tokens"] for r in recs] == [3, 4, 2]
    for p, r in zip([[5, 17, 3], [9, 8, 7, 6], [1, 2]], recs):
        assert r["tokens"] == plain.generate_greedy(pc, pt, p, 5, [3])
        assert r["finish_reason"] == ("length" if len(r["tokens"]) == 5 else "stop")
    outs = []
    for seed in ("4", "4", "5"):
        assert main(common + ["--temperature", "1.5", "--sample-seed", seed, "--prompt-ids", "5 17 3"],
                    ops=TorchOps(torch.float32)) == 0
        outs.append(capsys.readouterr().out)
    assert outs[0] == outs[1] and outs[0] != outs[2]
    with pytest.raises(SystemExit, match="nothing to generate"):
        main(common, ops=TorchOps(torch.float32))


@pytest.mark.parametrize("window", [None, 20])
def test_random_schedules_give_the_logits_of_whole_sequences(tmp_path, window):
    """Forty random ways of cutting and batching the same kind of work (requests of random lengths, each cut
    into steps of random sizes, run beside whatever else is live, in a cache so small that slots and
    pages are used again and, with a window, given back while a sequence still runs): the logits at
    every position are those of the whole sequence alone."""
    import random
    from rbitnet_b200 import StepEntry
    cfg = dict(TINY_A, sliding_window=window) if window else TINY_A
    folder = make_model_dir(tmp_path / "m", cfg, 3)
    ref = PlainModel(folder)
    from rbitnet_b200 import Engine
    eng = Engine.load_path(folder, dtype="float32", ops=TorchOps(torch.float32), max_tokens=256, page_size=16,
                           max_batch_tokens=37)
    rnd = random.Random(11)
    V, top = cfg["vocab_size"], cfg["max_position_embeddings"]
    for trial in range(40):
        n_req = rnd.randint(1, 4)
        reqs = [[rnd.randrange(V) for _ in range(rnd.choice([1, 2, 15, 16, 17, 33, 60]))] for _ in range(n_req)]
        reqs = [r[:min(len(r), 256 // n_req // 16 * 16, top)] for r in reqs]
        slots = [eng.new_sequence() for _ in reqs]
        done = [0] * n_req
        got = [[] for _ in reqs]
        while any(d < len(r) for d, r in zip(done, reqs)):
            entries, who = [], []
            for i, r in enumerate(reqs):
                if done[i] < len(r) and (rnd.random() < 0.7 or not entries):
                    n = min(len(r) - done[i], rnd.choice([1, 1, 2, 5, 16, 40]))
                    want = sorted(rnd.sample(range(n), rnd.randint(0, n)))
                    entries.append(StepEntry(slots[i], r[done[i]:done[i] + n], want))
                    who.append((i, done[i], want))
                    done[i] += n
            out = eng.step(entries)
            off = 0
            for i, base, want in who:
                for w in want:
                    got[i].append((base + w, out[off]))
                    off += 1
            assert (out is None and off == 0) or off == out.shape[0]
            for i in range(n_req):            # a finished request leaves at once; its slot and pages go to the next trial
                if done[i] == len(reqs[i]) and slots[i] is not None:
                    eng.end_sequence(slots[i])
                    slots[i] = None
        for i, r in enumerate(reqs):
            if got[i]:
                places = [p for p, _ in got[i]]
                assert_close(torch.stack([row for _, row in got[i]]), ref.logits(r)[places], "float32",
                             f"trial {trial} request {i}")
        assert eng.live_sequences() == []
    assert all(pool.n_free == pool.n for pool in eng.cache.book.pools)
