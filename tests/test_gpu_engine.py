"""The engine against the plain implementation, on the GPU, in 32-bit and in bfloat16:
whole requests; the last 32 tokens one by one; batches of unequal lengths whose shorter
requests end earlier, one batch after another so that slots are used again; long decoding;
the first tokens of a sequence; greedy generation through the entry point."""
import pytest
import torch

from helpers import assert_close, make_model_dir, PlainModel, TOL
from tiny import TINY_A, TINY_B, prompts
import plain_llama as plain

pytestmark = pytest.mark.gpu

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 2)}
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in CONFIGS.items():
        for store in DTYPES:
            out[name, store] = make_model_dir(tmp_path_factory.mktemp(f"tiny{name}_{store}"), cfg, seed, store)
    return out


@pytest.fixture(scope="module")
def engines(folders):
    from rbitnet_b200 import Engine
    made = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            made[key] = (Engine.load_path(folders[name, dtype], dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw),
                         PlainModel(folders[name, dtype]))
        return made[key]
    return get


def _cases():
    return [(n, d) for n in CONFIGS for d in DTYPES]


@pytest.mark.parametrize("name,dtype", _cases())
def test_whole_requests(engines, name, dtype):
    from rbitnet_b200 import StepEntry
    eng, ref = engines(name, dtype)
    V = eng.config.vocab_size
    for p in prompts([1, 2, 7, 33, 64, 65, 100], V, seed=5):
        s = eng.new_sequence()
        out = eng.step([StepEntry(s, p, list(range(len(p))))])
        eng.end_sequence(s)
        assert_close(out, ref.logits(p), dtype, f"whole len={len(p)}")


@pytest.mark.parametrize("name,dtype", _cases())
def test_last_32_one_by_one(engines, name, dtype):
    from rbitnet_b200 import StepEntry
    eng, ref = engines(name, dtype)
    V = eng.config.vocab_size
    for p in prompts([33, 80, 127], V, seed=6):
        s = eng.new_sequence()
        n0 = len(p) - 32
        outs = [eng.step([StepEntry(s, p[:n0], list(range(n0)))])]
        for t in p[n0:]:
            outs.append(eng.step([StepEntry(s, [t], [0])]))
        eng.end_sequence(s)
        assert_close(torch.cat(outs), ref.logits(p), dtype, f"tail32 len={len(p)}")


@pytest.mark.parametrize("name,dtype", _cases())
def test_unequal_batches_with_slot_reuse(engines, name, dtype):
    """Batches of unequal prompt and total lengths; shorter requests end earlier; three
    batches in a row on a cache that only holds one batch, so every slot and page is used again."""
    from rbitnet_b200 import StepEntry
    eng, ref = engines(name, dtype, max_tokens=512)
    V = eng.config.vocab_size
    plans = [([5, 9, 3, 70], [8, 2, 12, 5]), ([1, 17, 6, 11], [12, 12, 1, 7]), ([64, 2, 31, 16], [3, 9, 4, 20])]
    for b, (lens, decs) in enumerate(plans):
        ps = prompts([n + d for n, d in zip(lens, decs)], V, seed=20 + b)
        slots = [eng.new_sequence() for _ in ps]
        got = [[] for _ in ps]
        out = eng.step([StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(slots, ps, lens)])
        off = 0
        for i, n in enumerate(lens):
            got[i].append(out[off:off + n])
            off += n
        live = list(range(len(ps)))
        k = 0
        while live:
            out = eng.step([StepEntry(slots[i], [ps[i][lens[i] + k]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            k += 1
            for i in [i for i in live if decs[i] == k]:
                eng.end_sequence(slots[i])
            live = [i for i in live if decs[i] > k]
        for i, p in enumerate(ps):
            assert_close(torch.cat(got[i]), ref.logits(p), dtype, f"batch {b} request {i}")
    assert eng.live_sequences() == []
    assert all(pool.n_free == pool.n - 1 for pool in eng.cache.book.pools)     # all but the padding sequence's page


@pytest.mark.parametrize("name,dtype", _cases())
def test_long_decoding(engines, name, dtype):
    """One token at a time from the very first token up to the model's longest sequence."""
    from rbitnet_b200 import StepEntry
    eng, ref = engines(name, dtype)
    V, n = eng.config.vocab_size, eng.config.max_position_embeddings
    p = prompts([n], V, seed=8)[0]
    s = eng.new_sequence()
    outs = [eng.step([StepEntry(s, [t], [0])]) for t in p]
    eng.end_sequence(s)
    got, want = torch.cat(outs), ref.logits(p)
    assert_close(got[:4], want[:4], dtype, "first tokens")
    assert_close(got, want, dtype, "long decoding")


@pytest.mark.parametrize("name,dtype", _cases())
def test_context_overflow_is_refused(engines, name, dtype):
    from rbitnet_b200 import StepEntry
    from rbitnet_b200.cache import ContextOverflow
    eng, _ = engines(name, dtype)
    n = eng.config.max_position_embeddings
    s = eng.new_sequence()
    with pytest.raises(ContextOverflow):
        eng.step([StepEntry(s, [1] * (n + 1), [])])
    eng.end_sequence(s)


@pytest.mark.parametrize("name,dtype", _cases())
def test_a_far_key_among_hundreds(engines, name, dtype):
    """The answer depends on one early token only if attention reaches it: two sequences that
    differ in their first token alone must differ in their last logits as the plain model says."""
    from rbitnet_b200 import StepEntry
    eng, ref = engines(name, dtype)
    V, n = eng.config.vocab_size, eng.config.max_position_embeddings
    base = prompts([n], V, seed=9)[0]
    other = [(base[0] + 1) % V] + base[1:]
    outs = []
    for p in (base, other):
        s = eng.new_sequence()
        outs.append(eng.step([StepEntry(s, p, [n - 1])]))
        eng.end_sequence(s)
        assert_close(outs[-1], ref.logits(p)[-1:], dtype, "last logits")
    want = (ref.logits(base)[-1] - ref.logits(other)[-1])
    got = (outs[0][0] - outs[1][0]).double().cpu()
    if dtype == "float32":
        assert float(want.abs().max()) > 1e-4, "the plain model does not see the far key; test is void"
        assert float((got - want).abs().max()) <= 1e-5 + 1e-3 * float(want.abs().max())


@pytest.mark.parametrize("name,dtype", _cases())
def test_greedy_generation_through_the_entry_point(engines, name, dtype):
    eng, ref = engines(name, dtype)
    V = eng.config.vocab_size
    ps = prompts([4, 19, 1, 8, 30], V, seed=10)
    stop = [7]
    res = eng.generate(ps, max_tokens=10, temperature=0.0, stop_ids=stop, max_batch=3)
    assert eng.live_sequences() == []
    for p, r in zip(ps, res):
        # every emitted token must be the plain model's arg-max given the tokens before it
        # (within the dtype's tolerance at a near tie), and a stop token is never emitted
        seq = list(p)
        assert all(t not in stop for t in r.tokens)
        full = ref.logits(seq + r.tokens) if r.tokens else None
        for i, t in enumerate(r.tokens):
            row = full[len(p) - 1 + i]
            atol, rtol = TOL[dtype]
            assert float(row[t]) >= float(row.max()) - 2 * (atol + rtol * float(row.abs().max())), (i, t)
        if r.finish_reason == "length":
            assert len(r.tokens) == 10
        else:
            assert r.finish_reason == "stop" and len(r.tokens) < 10
    if dtype == "float32":
        for p, r in zip(ps, res):
            assert r.tokens == plain.generate_greedy(ref.cfg, ref.tensors, p, 10, stop)


# Mid-size configurations: head sizes 64 and 128 and widths of several tiles, so that the engine runs
# the tensor-core product over many tiles, the tcgen05 prefill attention and the split decode kernels
# (the tiny configurations have head sizes 16 and 32, which take the other attention kernels); then
# other head sizes, group sizes and a window, which take the remaining kernels and their masks.
MID = {
    "M64": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=512, num_attention_heads=8,
                num_key_value_heads=2, head_dim=64, intermediate_size=1432, vocab_size=1000, rope_theta=10000.0,
                rms_norm_eps=1e-5, max_position_embeddings=1024, tie_word_embeddings=False, rope_pairing="half"),
    "M128": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=768, num_attention_heads=6,
                 num_key_value_heads=3, head_dim=128, intermediate_size=1048, vocab_size=777, rope_theta=500000.0,
                 rms_norm_eps=1e-6, max_position_embeddings=1024, tie_word_embeddings=True,
                 rope_pairing="interleaved"),
    # head size 96, three query heads a group, an odd inner size: the mma.sync attention kernels
    "M96": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, hidden_size=576, num_attention_heads=6,
                num_key_value_heads=2, head_dim=96, intermediate_size=1111, vocab_size=900, rope_theta=1e6,
                rms_norm_eps=1e-5, max_position_embeddings=1024, tie_word_embeddings=False, rope_pairing="half"),
    # five query heads a group and a window of 100 keys in the tcgen05 prefill and the TMA-fed decode
    "M128w": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=1280, num_attention_heads=10,
                  num_key_value_heads=2, head_dim=128, intermediate_size=2056, vocab_size=1000, rope_theta=10000.0,
                  rms_norm_eps=1e-5, max_position_embeddings=1024, tie_word_embeddings=False, rope_pairing="half",
                  sliding_window=100),
    # one layer with the layer sizes of Llama-3-8B (the vocabulary is kept small: the plain model runs on the CPU)
    "L8B": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=1000, rope_theta=500000.0,
                rms_norm_eps=1e-5, max_position_embeddings=1024, tie_word_embeddings=False, rope_pairing="half"),
    # the largest head size
    "M256": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, hidden_size=768, num_attention_heads=3,
                 num_key_value_heads=1, head_dim=256, intermediate_size=304, vocab_size=300, rope_theta=10000.0,
                 rms_norm_eps=1e-6, max_position_embeddings=1024, tie_word_embeddings=True,
                 rope_pairing="interleaved"),
}


@pytest.mark.parametrize("name", list(MID))
@pytest.mark.parametrize("dtype", DTYPES)
def test_mid_size_prefill_chunks_and_decode(tmp_path, name, dtype):
    """Unequal prompts (one long enough for many key tiles) in one step, a second chunk for one of them,
    then tokens one by one for all; against the plain model."""
    from rbitnet_b200 import Engine, StepEntry
    cfg = MID[name]
    # q and k weights are scaled so that scores spread with a deviation of one at every width (it is
    # (0.02 * factor)^2 * hidden_size): 2.2 at a width of 512, 1.4 at 1280, 0.78 at 4096.  The bfloat16
    # band is stated for such scores: rounding q and k moves a score by 2^-9 of its size, so scores
    # twice as spread move the probabilities, and with them the logits, twice as far.
    import math
    folder = make_model_dir(tmp_path / "m", cfg, 11, store=dtype, factor=1.0 / (0.02 * math.sqrt(cfg["hidden_size"])))
    ref = PlainModel(folder)
    eng = Engine.load_path(folder, dtype=dtype, max_tokens=4096)
    V = cfg["vocab_size"]
    ps = prompts([700, 130, 37], V, seed=41)
    first = [520, 126, 33]
    slots = [eng.new_sequence() for _ in ps]
    got = [[] for _ in ps]
    out = eng.step([StepEntry(s, p[:n], [0, n // 2, n - 1]) for s, p, n in zip(slots, ps, first)])
    for i in range(3):
        got[i].append((out[3 * i:3 * i + 3], [0, first[i] // 2, first[i] - 1]))
    out = eng.step([StepEntry(slots[0], ps[0][520:696], [0, 175])])            # a later chunk of the long prompt
    got[0].append((out, [520, 695]))
    for k in range(4):
        out = eng.step([StepEntry(s, [p[len(p) - 4 + k]], [0]) for s, p in zip(slots, ps)])
        for i, p in enumerate(ps):
            got[i].append((out[i:i + 1], [len(p) - 4 + k]))
    for i, p in enumerate(ps):
        want = ref.logits(p)
        for rows, places in got[i]:
            assert_close(rows, want[places], dtype, f"{name} request {i} places {places}")
    for s in slots:
        eng.end_sequence(s)
    res = eng.generate([ps[1][:100], ps[2]], max_tokens=6, temperature=0.0)
    for p, r in zip([ps[1][:100], ps[2]], res):
        full = ref.logits(list(p) + r.tokens)
        for i, t in enumerate(r.tokens):
            row = full[len(p) - 1 + i]
            atol, rtol = TOL[dtype]
            assert float(row[t]) >= float(row.max()) - 2 * (atol + rtol * float(row.abs().max()))
