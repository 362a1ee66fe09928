"""The engine at the true layer sizes and vocabularies of the benchmark shapes (two layers each),
against the plain implementation, in 32-bit and in bfloat16, under the same three ways of cutting the
work as the tiny configurations: each request alone and whole; the last 32 tokens one by one; unequal
batches whose shorter requests end earlier, batch after batch on a cache that holds one batch.

The plain implementation runs in float64 with torch on the GPU here (on the CPU two layers of these
sizes take minutes); it is the same file, formula by formula
(crates/bitnet-core/src/llama/model.rs:219-316).  Weights are made on the device from (seed, name,
index), so nothing of these sizes is written to disk.
"""
import math

import pytest
import torch

from helpers import assert_close, sharpen, bf16_rtol
from tiny import prompts
import plain_llama as plain

pytestmark = pytest.mark.gpu

_BASE = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, rms_norm_eps=1e-5,
             tie_word_embeddings=False, rope_pairing="half", hidden_act="silu", max_position_embeddings=2048)
SHAPES = {
    # Llama-3-8B: grouped queries 4:1, head size 128
    "llama3_8b": dict(_BASE, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      intermediate_size=14336, vocab_size=128256, rope_theta=500000.0),
    # Llama-2-7B: one kv head per query head
    "llama2_7b": dict(_BASE, hidden_size=4096, num_attention_heads=32, num_key_value_heads=32, head_dim=128,
                      intermediate_size=11008, vocab_size=32000, rope_theta=10000.0),
    # TinyLlama-1.1B: grouped queries 8:1, head size 64
    "tinyllama": dict(_BASE, hidden_size=2048, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                      intermediate_size=5632, vocab_size=32000, rope_theta=10000.0),
}
DTYPES = ["float32", "bfloat16"]


def _tensors(cfg, seed, store):
    """Random weights on the device; q and k scaled so that scores spread with a deviation of about one."""
    from rbitnet_b200.config import config_from_dict
    from rbitnet_b200.config.registry import get_architecture
    from rbitnet_b200.weights import random_tensors
    c = config_from_dict(cfg)
    spec = get_architecture(c.architecture).build_spec(c)
    t = random_tensors(spec, seed, device="cuda")
    t = sharpen(t, 1.0 / (0.02 * math.sqrt(cfg["hidden_size"])))
    return c, {k: v.to({"float32": torch.float32, "bfloat16": torch.bfloat16}[store]) for k, v in t.items()}


class _Oracle:
    def __init__(self, cfg, tensors):
        self.cfg, self.tensors, self._memo = cfg, tensors, {}

    def logits(self, tokens, rows):
        key = tuple(tokens)
        if key not in self._memo:
            self._memo = {key: plain.forward(self.cfg, self.tensors, list(tokens), torch.float64)}   # keep one: they are large
        return self._memo[key][torch.as_tensor(rows, device="cuda")].cpu()


@pytest.fixture(scope="module")
def made():
    cache = {}

    def get(name, dtype):
        from rbitnet_b200 import Engine
        key = (name, dtype)
        if key not in cache:
            cache.clear()          # one model of these sizes at a time
            torch.cuda.empty_cache()
            cfg, tensors = _tensors(SHAPES[name], 21, dtype)
            eng = Engine(cfg, dict(tensors), dtype=dtype, max_tokens=640, max_seq=512)
            cache[key] = (eng, _Oracle(SHAPES[name], tensors))
        return cache[key]
    yield get
    cache.clear()
    torch.cuda.empty_cache()


def _cases():
    return [(n, d) for n in SHAPES for d in DTYPES]


@pytest.mark.parametrize("name,dtype", _cases())
def test_whole_tail_and_unequal_batches(made, name, dtype):
    from rbitnet_b200 import StepEntry
    eng, ref = made(name, dtype)
    V = SHAPES[name]["vocab_size"]
    L = SHAPES[name]["num_hidden_layers"]
    rtol = bf16_rtol(L) if dtype == "bfloat16" else None
    reqs = prompts([97, 150, 40, 131, 66], V, seed=77)
    # ---- each request alone and whole
    for p in reqs[:3]:
        n = len(p)
        want = sorted({0, 1, n // 3, n // 2, n - 2, n - 1})
        s = eng.new_sequence()
        out = eng.step([StepEntry(s, p, want)])
        eng.end_sequence(s)
        assert_close(out, ref.logits(p, want), dtype, f"{name} whole len={n}", rtol=rtol)
    # ---- the last 32 tokens one by one (the captured decode step for half of them)
    for p in reqs[1:3]:
        n0 = len(p) - 32
        s = eng.new_sequence()
        outs = [eng.step([StepEntry(s, p[:n0], [0, n0 - 1])])]
        for k, t in enumerate(p[n0:]):
            outs.append(eng.step([StepEntry(s, [t], [0])], captured=k % 2 == 1))
        eng.end_sequence(s)
        assert_close(torch.cat(outs), ref.logits(p, [0, n0 - 1] + list(range(n0, len(p)))), dtype,
                     f"{name} tail32 len={len(p)}", rtol=rtol)
    # ---- unequal batches, shorter requests end earlier, two batches on a cache that holds one
    plans = [([0, 1, 2], [80, 140, 30]), ([3, 4, 0], [120, 50, 90])]
    for b, (which, lens) in enumerate(plans):
        ps = [reqs[i] for i in which]
        slots = [eng.new_sequence() for _ in ps]
        got = [[] for _ in ps]
        places = [[0, n - 1] for n in lens]
        out = eng.step([StepEntry(s, p[:n], [0, n - 1]) for s, p, n in zip(slots, ps, lens)])
        for i in range(len(ps)):
            got[i].append(out[2 * i:2 * i + 2])
        live, k = list(range(len(ps))), 0
        while live:
            out = eng.step([StepEntry(slots[i], [ps[i][lens[i] + k]], [0]) for i in live], captured=k % 2 == 0)
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                places[i].append(lens[i] + k)
            k += 1
            for i in [i for i in live if lens[i] + k == len(ps[i])]:
                eng.end_sequence(slots[i])
            live = [i for i in live if lens[i] + k < len(ps[i])]
        for i, p in enumerate(ps):
            assert_close(torch.cat(got[i]), ref.logits(p, places[i]), dtype, f"{name} batch {b} request {i}", rtol=rtol)
    assert eng.live_sequences() == []


def test_bfloat16_against_float32_at_eight_layers():
    """Eight layers of the Llama-3-8B shape: the bfloat16 engine against this library's own float32
    engine on the same weights (a prompt, then tokens one by one), within the band for eight layers."""
    from rbitnet_b200 import Engine, StepEntry
    cfg = dict(SHAPES["llama3_8b"], num_hidden_layers=8)
    c, tensors = _tensors(cfg, 5, "bfloat16")       # both engines read the same bfloat16 weights
    p = prompts([150], cfg["vocab_size"], seed=3)[0]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(c, dict(tensors), dtype=dtype, max_tokens=256, max_seq=256)
        s = eng.new_sequence()
        rows = [eng.step([StepEntry(s, p[:140], [0, 70, 139])])]
        for t in p[140:]:
            rows.append(eng.step([StepEntry(s, [t], [0])], captured=True))
        outs[dtype] = torch.cat(rows).double().cpu()
        eng.end_sequence(s)
        del eng
        torch.cuda.empty_cache()
    assert_close(outs["bfloat16"], outs["float32"], "bfloat16", "8 layers, bfloat16 against float32", rtol=bf16_rtol(8))
    agree = (outs["bfloat16"].argmax(1) == outs["float32"].argmax(1)).float().mean()
    assert agree >= 0.5, f"only {agree:.2f} of the arg-max agree"


@pytest.mark.parametrize("name", ["llama3_8b", "tinyllama"])
def test_a_decode_steps_norms_in_the_products_around_them_or_as_kernels(made, name):
    """Up to 16 tokens a step's norms between two products ride in those products: two kernels fewer per
    layer (but for the first layer's first norm), and logits that differ from the same step with every norm
    a kernel only by where bfloat16 rounds (row x weight, or row x factor x weight)."""
    from rbitnet_b200 import StepEntry
    eng, ref = made(name, "bfloat16")
    L = SHAPES[name]["num_hidden_layers"]
    p = prompts([60], SHAPES[name]["vocab_size"], seed=9)[0]
    got, launches = {}, {}
    try:
        for fold in (True, False):
            eng.ops.fold_norms = fold
            s = eng.new_sequence()
            eng.step([StepEntry(s, p[:40], [])])
            rows = []
            for t in p[40:]:
                before = eng.ops.lib.launches
                rows.append(eng.step([StepEntry(s, [t], [0])]))           # (not captured: a captured step keeps its path)
                launches[fold] = eng.ops.lib.launches - before
            eng.end_sequence(s)
            got[fold] = torch.cat(rows)
    finally:
        eng.ops.fold_norms = True
    assert launches[False] - launches[True] == 2 * L - 1, launches
    want = ref.logits(p, list(range(40, 60)))
    assert_close(got[True], want, "bfloat16", f"{name} folded norms", rtol=bf16_rtol(L))
    assert_close(got[False], want, "bfloat16", f"{name} norms as kernels", rtol=bf16_rtol(L))
    assert_close(got[True], got[False].double().cpu(), "bfloat16", f"{name} folded against kernels", rtol=bf16_rtol(L))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_of_the_benchmark_s_length_at_the_benchmark_s_layer_sizes(dtype):
    """2,048 tokens in one step at the Llama-3-8B layer sizes (two layers), then three tokens one by one: the
    products of many tokens (tiles that leave as TMA boxes, weight tiles shared between teams of CTAs) and
    the tcgen05 attention over 16 key tiles, against the plain model in float64 at places all along the
    prompt."""
    from rbitnet_b200 import Engine, StepEntry
    cfg = dict(SHAPES["llama3_8b"], max_position_embeddings=4096)
    c, tensors = _tensors(cfg, 33, dtype)
    p = prompts([2051], cfg["vocab_size"], seed=5)[0]
    eng = Engine(c, dict(tensors), dtype=dtype, max_tokens=2304, max_seq=2304)
    s = eng.new_sequence()
    places = [0, 1, 127, 128, 255, 256, 1000, 1023, 1024, 1500, 2046, 2047]
    rows = [eng.step([StepEntry(s, p[:2048], places)])]
    for t in p[2048:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]))
    eng.end_sequence(s)
    got = torch.cat(rows).double().cpu()
    del eng
    torch.cuda.empty_cache()
    want = plain.forward(cfg, tensors, list(p), torch.float64)[torch.as_tensor(places + [2048, 2049, 2050], device="cuda")].cpu()
    rtol = bf16_rtol(cfg["num_hidden_layers"]) if dtype == "bfloat16" else None
    assert_close(got, want, dtype, "2,048 tokens at the 8B layer sizes", rtol=rtol)


def test_one_prompt_cut_into_steps_in_seven_ways_at_the_benchmark_s_layer_sizes():
    """1,500 tokens of the Llama-3-8B layer sizes (two layers, bfloat16) whole, and cut so that the cuts
    fall on both sides of every choice the products make (tiles of 16 and 64, 257 tokens, shared weight
    tiles, one token at the end): the logits at the last position against the plain model in float64."""
    from rbitnet_b200 import Engine, StepEntry
    cfg = dict(SHAPES["llama3_8b"], max_position_embeddings=4096)
    c, tensors = _tensors(cfg, 33, "bfloat16")
    eng = Engine(c, dict(tensors), dtype="bfloat16", max_tokens=4096, max_seq=2304)
    p = prompts([1500], cfg["vocab_size"], seed=8)[0]
    want = plain.forward(cfg, tensors, list(p), torch.float64)[-1:].cpu()
    ways = ([1500], [300, 1200], [700, 800], [64] * 23 + [28], [257, 256, 255, 732], [1499, 1], [1000, 499, 1],
            [16] * 93 + [12])
    for cuts in ways:
        s, at, out = eng.new_sequence(), 0, None
        for n in cuts:
            out = eng.step([StepEntry(s, p[at:at + n], [n - 1])])
            at += n
        eng.end_sequence(s)
        assert_close(out, want, "bfloat16", f"cut as {cuts[:4]}... ({len(cuts)} steps)", rtol=bf16_rtol(cfg["num_hidden_layers"]))
