"""Paths of the engine that the plain step-by-step tests do not reach: the captured decode step's
own logits (padding rows, page edges, a moving window edge, slots used again), temperature sampling
through ``Engine.generate``, a cache that a batch fills to the last page, the ``generate`` verb of
the command line, the kernels' error word on its way to an exception, and the weight modes."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import assert_close, make_model_dir, PlainModel
from tiny import TINY_A, TINY_B, prompts
import plain_llama as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 2)}
DTYPES = ["float32", "bfloat16"]

# a windowed two-layer model with head size 128 (the tcgen05 prefill, the TMA-fed split decode)
WINDOWED = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=512, num_attention_heads=4,
                num_key_value_heads=2, head_dim=128, intermediate_size=1032, vocab_size=500, rope_theta=10000.0,
                rms_norm_eps=1e-5, max_position_embeddings=512, tie_word_embeddings=False, rope_pairing="half",
                sliding_window=50)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in CONFIGS.items():
        for store in DTYPES:
            out[name, store] = make_model_dir(tmp_path_factory.mktemp(f"s{name}_{store}"), cfg, seed, store)
    for store in DTYPES:
        out["W", store] = make_model_dir(tmp_path_factory.mktemp(f"sW_{store}"), WINDOWED, 4, store, factor=2.0)
    return out


def _cases(names=("A", "B")):
    return [(n, d) for n in names for d in DTYPES]


# --------------------------------------------------------------------------- the captured step's logits
@pytest.mark.parametrize("name,dtype", _cases(("A", "B", "W")))
def test_captured_steps_across_page_and_window_edges(folders, name, dtype):
    """Three sequences (so the captured step of four has a padding row) decode 70 tokens one by one
    from prompts of about 60 tokens: every sequence gets a second page after the step was captured,
    and in the windowed model the window's edge moves with every step.  The captured step's logits
    are compared with the plain model at every step; then the same again on the freed slots."""
    from rbitnet_b200 import Engine, StepEntry
    eng = Engine.load_path(folders[name, dtype], dtype=dtype, max_tokens=3 * 192)
    ref = PlainModel(folders[name, dtype])
    V = eng.config.vocab_size
    top = min(eng.config.max_position_embeddings, 190)
    for round_ in range(2):
        lens = [58, 61, 63] if round_ == 0 else [63, 5, 60]
        ps = prompts([min(top, n + 70) for n in lens], V, seed=30 + round_)
        slots = [eng.new_sequence() for _ in ps]
        got = [[] for _ in ps]
        out = eng.step([StepEntry(s, p[:n], [n - 1]) for s, p, n in zip(slots, ps, lens)])
        for i in range(3):
            got[i].append(out[i:i + 1])
        live, k = [0, 1, 2], 0
        while live:
            out = eng.step([StepEntry(slots[i], [ps[i][lens[i] + k]], [0]) for i in live], captured=True)
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            k += 1
            for i in [i for i in live if lens[i] + k == len(ps[i])]:
                eng.end_sequence(slots[i])
            live = [i for i in live if lens[i] + k < len(ps[i])]
        for i, p in enumerate(ps):
            assert_close(torch.cat(got[i]), ref.logits(p)[lens[i] - 1:], dtype, f"{name} round {round_} request {i}")
    assert eng.live_sequences() == []
    assert 4 in eng._graphs and eng._graphs[4].graph is not None        # the step of 3 ran as the graph of 4


@pytest.mark.parametrize("name,dtype", _cases())
@pytest.mark.parametrize("batch", [3, 5, 7])
def test_captured_step_equals_the_step_function(folders, name, dtype, batch):
    """The same decode steps through the captured graph and kernel by kernel: same logits, whatever
    the number of padding rows (batches of 3, 5 and 7 run as graphs of 4, 8 and 8)."""
    from rbitnet_b200 import Engine, StepEntry
    V = CONFIGS[name][0]["vocab_size"]
    lens = [3, 17, 9, 30, 1, 12, 25][:batch]
    ps = prompts([n + 6 for n in lens], V, seed=50 + batch)
    outs = {}
    for captured in (False, True):
        eng = Engine.load_path(folders[name, dtype], dtype=dtype, max_tokens=batch * 64)
        slots = [eng.new_sequence() for _ in ps]
        eng.step([StepEntry(s, p[:n], []) for s, p, n in zip(slots, ps, lens)])
        rows = []
        for k in range(6):
            want = [[0] if (i + k) % 3 else [] for i in range(batch)]          # some rows are not asked for
            rows.append(eng.step([StepEntry(s, [p[n + k]], w) for s, p, n, w in zip(slots, ps, lens, want)],
                                 captured=captured))
        outs[captured] = torch.cat(rows)
        for s in slots:
            eng.end_sequence(s)
    assert outs[True].shape == outs[False].shape
    if dtype == "float32":
        assert float((outs[True] - outs[False]).abs().max()) <= 1e-5
    else:       # other numbers of splits of K and of the keys: other roundings
        assert_close(outs[True], outs[False].double().cpu(), dtype, "captured against step by step")


# --------------------------------------------------------------------------- sampling through the engine
@pytest.mark.parametrize("name", ["A", "B"])
def test_temperature_generation_follows_the_plain_model_and_ignores_batching(folders, name):
    """crates/bitnet-core/src/llama/runtime.rs:94-106 with the draw u(seed, request, step): every
    emitted token is the plain model's choice for that draw given the tokens so far, and the ids do
    not depend on how the requests were batched."""
    from rbitnet_b200 import Engine
    from rbitnet_b200.sampling.rng import uniform
    eng = Engine.load_path(folders[name, "float32"], dtype="float32", max_tokens=1024)
    ref = PlainModel(folders[name, "float32"])
    V = eng.config.vocab_size
    ps = prompts([4, 19, 1, 8, 30], V, seed=12)
    T, seed, n_new = 0.8, 1234, 9
    base = eng.generate(ps, max_tokens=n_new, temperature=T, seed=seed, stop_ids=[], max_batch=5)
    for r, (p, res) in enumerate(zip(ps, base)):
        assert len(res.tokens) == n_new and res.finish_reason == "length"
        full = ref.logits(list(p) + res.tokens)
        for i, t in enumerate(res.tokens):
            row = full[len(p) - 1 + i]
            u = uniform(seed, r, i)
            want = plain.temperature_token(row, T, u)
            if t != want:
                # the draw may land within float32 rounding of a boundary of the cumulative sum
                c = plain.temperature_cdf(row, T)
                edge = float(c[min(t, want)]) / float(c[-1])
                assert abs(t - want) == 1 and abs(edge - u) < 1e-5, (r, i, t, want, edge, u)
    assert len({tuple(r.tokens) for r in base}) > 1
    for mb in (1, 3):
        again = eng.generate(ps, max_tokens=n_new, temperature=T, seed=seed, stop_ids=[], max_batch=mb)
        assert [r.tokens for r in again] == [r.tokens for r in base], f"max_batch={mb}"
    other = eng.generate(ps, max_tokens=n_new, temperature=T, seed=seed + 1, stop_ids=[])
    assert [r.tokens for r in other] != [r.tokens for r in base]
    assert eng.live_sequences() == []


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_that_fills_the_cache_to_its_last_page(folders, dtype):
    """Three requests that grow to 64, 64 and 70 positions in a cache of exactly four pages; each
    holds one page after its prompt and the third needs its second page in the middle of decoding.
    The captured step of four has a padding row; the padding sequence has a page of its own and
    takes none of theirs."""
    from rbitnet_b200 import Engine
    eng = Engine.load_path(folders["A", dtype], dtype=dtype, max_tokens=256)
    ref = PlainModel(folders["A", dtype])
    ps = prompts([54, 54, 60], 256, seed=13)
    res = eng.generate(ps, max_tokens=10, temperature=0.0, stop_ids=[], max_batch=3)
    assert [len(r.tokens) for r in res] == [10, 10, 10] and all(r.finish_reason == "length" for r in res)
    assert eng.last_stats["steps"] == 10            # one batch: nobody had to wait for a page
    if dtype == "float32":
        for p, r in zip(ps, res):
            assert r.tokens == plain.generate_greedy(ref.cfg, ref.tensors, p, 10)
    assert eng.live_sequences() == []
    assert all(pool.n_free == pool.n - 1 for pool in eng.cache.book.pools)      # all but the padding sequence's page


# --------------------------------------------------------------------------- command line
def test_generate_verb_of_the_command_line(tmp_path):
    """``python -m rbitnet_b200 random`` then ``generate --prompt-ids ... --temperature 0`` as a user
    runs them; the printed ids are the plain model's greedy ids."""
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(TINY_B))
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    model = tmp_path / "model"
    p = subprocess.run([sys.executable, "-m", "rbitnet_b200", "random", "--config", str(cfg_file), "--out", str(model),
                        "--seed", "5", "--dtype", "float32"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ps = prompts([7, 3], TINY_B["vocab_size"], seed=14)
    cmd = [sys.executable, "-m", "rbitnet_b200", "generate", "--model", str(model), "--dtype", "float32",
           "--temperature", "0", "--max-tokens", "8", "--stop-id", "3", "--cache-tokens", "512"]
    for q in ps:
        cmd += ["--prompt-ids", " ".join(map(str, q))]
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [json.loads(x) for x in p.stdout.strip().splitlines()]
    pc, pt = plain.load_folder(model)
    assert len(lines) == 2
    for q, rec in zip(ps, lines):
        assert rec["tokens"] == plain.generate_greedy(pc, pt, q, 8, [3])
        assert rec["prompt_tokens"] == len(q)


# --------------------------------------------------------------------------- the error word
def test_error_word_reaches_the_caller_and_leaves_nothing_behind(folders):
    """crates/bitnet-core/src/llama/model.rs:221-227 and crates/bitnet-core/src/error.rs:5-29 are the
    reference's typed errors on the forward path; here a kernel whose bounded wait ran out records a
    code in a device word.  The word is written from the host (no kernel waits for anything): the
    next step, captured or not, raises with the code, the word is clear afterwards, and the
    generation loop has given every slot back."""
    from rbitnet_b200 import Engine, StepEntry
    from rbitnet_b200.kernels.lib import KernelError
    eng = Engine.load_path(folders["A", "bfloat16"], dtype="bfloat16", max_tokens=512)
    ps = prompts([5, 9, 3], 256, seed=15)
    assert [len(r.tokens) for r in eng.generate(ps, max_tokens=4, temperature=0.0, stop_ids=[])] == [4, 4, 4]
    lib = eng.ops.lib
    lib.call("rb_set_error_flag_for_test", 2, launches=0)
    with pytest.raises(KernelError, match="code 2"):
        eng.generate(ps, max_tokens=4, temperature=0.0, stop_ids=[])
    assert eng.live_sequences() == []
    eng.ops.check_errors()                                      # clear again
    lib.call("rb_set_error_flag_for_test", 3, launches=0)
    s = eng.new_sequence()
    eng.step([StepEntry(s, ps[0], [0])])                        # the step function itself does not read the word ...
    with pytest.raises(KernelError, match="code 3"):
        eng.ops.check_errors()                                  # ... the caller asks
    eng.ops.check_errors()
    with pytest.raises(KernelError, match="code 2"):            # the captured step brings the word back itself
        lib.call("rb_set_error_flag_for_test", 2, launches=0)
        eng.step([StepEntry(s, [1], [0])], captured=True)
    eng.ops.check_errors()
    eng.end_sequence(s)
    assert [len(r.tokens) for r in eng.generate(ps, max_tokens=4, temperature=0.0, stop_ids=[])] == [4, 4, 4]


def test_a_bounded_wait_gives_up_and_says_so():
    """The wait the tensor-core kernels use, on a barrier at which nobody arrives, in a kernel that does
    nothing else and with a limit of a millisecond: it returns, and the word holds its code."""
    import ctypes
    import time
    from rbitnet_b200.kernels.ops import CudaOps
    from rbitnet_b200.kernels.lib import KernelError
    ops = CudaOps(torch.bfloat16)
    ops.check_errors()
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    ops.lib.call("rb_wait_probe", 1_000_000, 7, ctypes.c_void_p(gave_up.data_ptr()), ops._stream())
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert int(gave_up[0]) == 1
    with pytest.raises(KernelError, match="code 7"):
        ops.check_errors()
    ops.check_errors()                                          # cleared by the read above
    with pytest.raises(KernelError, match="at most 0.1 s"):
        ops.lib.call("rb_wait_probe", 3_000_000_000, 7, ctypes.c_void_p(gave_up.data_ptr()), ops._stream())
    # the wait on a count in global memory (the finished parts of a shared weight tile), same limit, same word
    zero = torch.zeros(1, dtype=torch.int32, device="cuda")
    gave_up.zero_()
    t0 = time.time()
    ops.lib.call("rb_count_wait_probe", ctypes.c_void_p(zero.data_ptr()), 1_000_000, 4,
                 ctypes.c_void_p(gave_up.data_ptr()), ops._stream())
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0 and int(gave_up[0]) == 1
    with pytest.raises(KernelError, match="code 4"):
        ops.check_errors()
    ops.check_errors()
    # the context is as usable as before
    assert int((torch.ones(4, device="cuda") * 2).sum()) == 8


# --------------------------------------------------------------------------- weights
def test_random_weights_are_the_same_on_both_devices_and_through_a_folder(tmp_path):
    """crates/bitnet-core/src/model/toy.rs:16-30: one seed, one model, wherever it is made."""
    from rbitnet_b200 import Engine, StepEntry, write_random_model
    from rbitnet_b200.config import config_from_dict
    from rbitnet_b200.weights import random_tensor
    a = random_tensor("model.layers.0.mlp.up_proj.weight", (300, 41), "matrix", 3, device="cuda")
    b = random_tensor("model.layers.0.mlp.up_proj.weight", (300, 41), "matrix", 3, device="cpu")
    assert torch.equal(a.cpu(), b)
    cfg = config_from_dict(TINY_B)
    folder = write_random_model(tmp_path / "m", cfg, seed=9)
    p = prompts([20], cfg.vocab_size, seed=16)[0]
    outs = []
    for eng in (Engine.from_random(cfg, 9, dtype="float32", max_tokens=256),
                Engine.load_path(folder, dtype="float32", max_tokens=256)):
        s = eng.new_sequence()
        outs.append(eng.step([StepEntry(s, p, list(range(len(p))))]))
        eng.end_sequence(s)
    assert torch.equal(outs[0], outs[1])


def test_a_half_precision_folder_is_exact_in_float32_and_harmless_extras_load(tmp_path):
    """Weights stored as F16 reach the float32 engine unrounded; a folder that also holds
    ``rotary_emb.inv_freq`` buffers (as older exports do) loads, with a warning."""
    from rbitnet_b200 import Engine, StepEntry
    from rbitnet_b200.config import config_from_dict
    from rbitnet_b200.config.registry import get_architecture
    from rbitnet_b200.weights import random_tensors, write_safetensors
    from helpers import sharpen
    cfg = config_from_dict(TINY_A)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = {k: v.to(torch.float16) for k, v in sharpen(random_tensors(spec, 8), 4.0).items()}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8, dtype=torch.float32)
    folder = tmp_path / "half"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.warns(UserWarning, match="inv_freq"):
        eng = Engine.load_path(folder, dtype="float32", max_tokens=256)
    del tensors["model.layers.0.self_attn.rotary_emb.inv_freq"]
    p = prompts([40], 256, seed=17)[0]
    s = eng.new_sequence()
    out = eng.step([StepEntry(s, p, list(range(len(p))))])
    eng.end_sequence(s)
    want = plain.forward(TINY_A, tensors, p, torch.float64)       # the F16 values, exactly
    assert_close(out, want, "float32", "F16 folder in float32")
    rounded = plain.forward(TINY_A, {k: v.to(torch.bfloat16) for k, v in tensors.items()}, p, torch.float64)
    assert float((rounded - want).abs().max()) > 20 * float((out.double().cpu() - want).abs().max())


# --------------------------------------------------------------------------- the checked build
_CHECKED_SCRIPT = r'''
import sys, json, math, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from rbitnet_b200.kernels.ops import CudaOps
from rbitnet_b200.kernels.lib import KernelError
from rbitnet_b200.cache import CacheLayerView
from rbitnet_b200 import Engine
import plain_llama as plain
from tiny import prompts

ops = CudaOps(torch.float32)
assert ops.lib.raw("rb_is_checked_build")() == 1
# a whole model runs in the checked build and nothing is recorded
eng = Engine.load_path(sys.argv[2], dtype="float32", max_tokens=512)
pc, pt = plain.load_folder(sys.argv[2])
ps = prompts([5, 70], pc["vocab_size"], seed=3)
res = eng.generate(ps, max_tokens=6, temperature=0.0, stop_ids=[])
assert [r.tokens for r in res] == [plain.generate_greedy(pc, pt, p, 6) for p in ps]
ops.check_errors()
# one token at a position past its slot's row of the page table: 8 pages of 16 positions, position 128.
# (Entry 8 of slot 0's row is entry 0 of slot 1's row, so even the unchecked address would lie inside
# the cache; the checked build records it and does not use it.)
H, Kh, D, page, max_pages, n_slots = 2, 1, 16, 16, 8, 4
k = torch.zeros(n_slots * max_pages, Kh, page, D, device="cuda")
v = torch.zeros_like(k)
table = torch.arange(n_slots * max_pages, dtype=torch.int32, device="cuda").reshape(n_slots, max_pages)
view = CacheLayerView(k, v, table, max_pages, page, Kh, D, True, 0)
class M: pass
m = M()
m.tok_slot = torch.tensor([0, 0], dtype=torch.int32, device="cuda")
m.tok_pos = torch.tensor([5, 128], dtype=torch.int32, device="cuda")
qkv = torch.ones(2, (H + 2 * Kh) * D, device="cuda")
inv = torch.zeros(D // 2, device="cuda")
ops.rotate_append(qkv, (inv, False, D), m, view, H)
torch.cuda.synchronize()
try:
    ops.check_errors()
    print("NOT RECORDED")
except KernelError as e:
    print("RECORDED", e)
ops.check_errors()                       # cleared
assert float(k[8].abs().sum()) == 0      # slot 1's first page was not touched
assert float(k[0, 0, 5].abs().sum()) > 0 # the good token was appended
print("OK")
'''


def test_checked_build_records_a_bad_cache_address_and_does_not_use_it(folders, tmp_path):
    """The library built with RBITNET_CHECKED=1 (its own shared object, compiled at first use) runs a
    model like the plain build, and a position outside a sequence's page-table row is recorded with
    its slot and position instead of being used."""
    script = tmp_path / "checked.py"
    script.write_text(_CHECKED_SCRIPT)
    env = dict(os.environ, RBITNET_CHECKED="1", PYTHONPATH="")
    p = subprocess.run([sys.executable, str(script), str(ROOT), str(folders["A", "float32"])], capture_output=True,
                       text=True, env=env, timeout=900)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert "RECORDED" in p.stdout and "slot 0, position 128" in p.stdout and p.stdout.strip().endswith("OK"), p.stdout


# --------------------------------------------------------------------------- random ways of cutting the work
@pytest.mark.parametrize("name,dtype", _cases(("B", "W")))
def test_random_schedules_give_the_logits_of_whole_sequences(folders, name, dtype):
    """Random requests cut into steps of random sizes, run beside whatever else is live, some steps through
    the captured decode step, in a cache small enough that slots and pages are used again (and, in the
    windowed model, given back while a sequence still runs): every logit is that of its whole sequence."""
    import random
    from rbitnet_b200 import Engine, StepEntry
    eng = Engine.load_path(folders[name, dtype], dtype=dtype, max_tokens=4 * 256, max_batch_tokens=150)
    ref = PlainModel(folders[name, dtype])
    rnd = random.Random(23)
    V, top = eng.config.vocab_size, min(eng.config.max_position_embeddings, 256)
    for trial in range(12):
        n_req = rnd.randint(1, 4)
        reqs = [[rnd.randrange(V) for _ in range(min(top, rnd.choice([1, 2, 63, 64, 65, 130, 200])))] for _ in range(n_req)]
        slots = [eng.new_sequence() for _ in reqs]
        done = [0] * n_req
        got = [[] for _ in reqs]
        while any(d < len(r) for d, r in zip(done, reqs)):
            entries, who = [], []
            single = rnd.random() < 0.5
            for i, r in enumerate(reqs):
                if done[i] < len(r) and (rnd.random() < 0.7 or not entries):
                    n = 1 if single else min(len(r) - done[i], rnd.choice([1, 2, 7, 64, 100]))
                    want = sorted(rnd.sample(range(n), rnd.randint(0 if not single else 1, n)))
                    entries.append(StepEntry(slots[i], r[done[i]:done[i] + n], want))
                    who.append((i, done[i], want))
                    done[i] += n
            out = eng.step(entries, captured=single and rnd.random() < 0.7)
            off = 0
            for i, base, want in who:
                for w in want:
                    got[i].append((base + w, out[off].clone()))
                    off += 1
            for i in range(n_req):
                if done[i] == len(reqs[i]) and slots[i] is not None:
                    eng.end_sequence(slots[i])
                    slots[i] = None
        for i, r in enumerate(reqs):
            if got[i]:
                places = [p for p, _ in got[i]]
                assert_close(torch.stack([row for _, row in got[i]]), ref.logits(r)[places], dtype,
                             f"{name} trial {trial} request {i}")
        assert eng.live_sequences() == []
