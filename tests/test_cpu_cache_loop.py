"""The cache's bookkeeping and the generation loop's decisions (no GPU)."""
import random

import pytest
import torch

from rbitnet_b200.cache import (FreeList, SlotBook, CacheFull, ContextOverflow, SequenceCache)
from rbitnet_b200.parts import CacheNeed, StateNeed
from rbitnet_b200.engine import GenerationLoop
from rbitnet_b200.sampling import uniform


def test_free_list_never_loses_or_doubles():
    f = FreeList(5)
    got = [f.take() for _ in range(5)]
    assert sorted(got) == list(range(5))
    with pytest.raises(CacheFull):
        f.take()
    f.give(3)
    with pytest.raises(ValueError, match="not held"):
        f.give(3)
    with pytest.raises(ValueError, match="not held"):
        f.give(99)
    assert f.take() == 3


def test_slot_book_random_walk_keeps_every_page_accounted_for():
    rng = random.Random(0)
    book = SlotBook(n_slots=6, pages_per_group=[20, 20], page_size=16, max_seq=100)
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            s = book.alloc()
            assert s not in live
            live[s] = 0
        elif op < 0.4 and live:
            s = rng.choice(sorted(live))
            book.free(s)
            del live[s]
        elif live:
            s = rng.choice(sorted(live))
            n = rng.randint(1, 40)
            try:
                book.reserve(s, n)
                book.advance(s, n)
                live[s] += n
            except (CacheFull, ContextOverflow):
                pass
        # invariants: no page held twice, none lost, lengths right
        for g, pool in enumerate(book.pools):
            held = [p for s in live for p in book.pages[s][g]]
            assert len(held) == len(set(held))
            assert set(held) == set(pool.held)
            assert pool.n_free + len(held) == pool.n
        for s, n in live.items():
            assert book.length[s] == n
            assert all(len(pg) * 16 >= n for pg in book.pages[s])
        assert book.slots.n_free + len(live) == 6
    for s in list(live):
        book.free(s)
    assert all(p.n_free == p.n for p in book.pools)


def test_slot_book_errors():
    book = SlotBook(2, [4], 16, 50)
    a = book.alloc()
    with pytest.raises(ContextOverflow):
        book.reserve(a, 51)
    book.reserve(a, 50)                      # 4 pages
    b = book.alloc()
    with pytest.raises(CacheFull):
        book.reserve(b, 1)
    assert book.pools[0].n_free == 0 and book.pages[b] == [[]]   # a failed reserve keeps nothing
    with pytest.raises(CacheFull, match="slots"):
        book.alloc()
    book.free(a)
    with pytest.raises(ValueError, match="not live"):
        book.free(a)
    with pytest.raises(ValueError):
        book.advance(b, 17)
    book.reserve(b, 1)
    book.advance(b, 1)


def test_sequence_cache_groups_views_and_state():
    needs = {0: CacheNeed(2, 16), 1: CacheNeed(2, 16, window=8), 2: CacheNeed(2, 16)}
    cache = SequenceCache(needs, reads={3: 0}, state_needs={1: StateNeed((5,), torch.float32)},
                          max_tokens=256, max_seq=128, dtype=torch.float32, device="cpu", page_size=16)
    assert len(cache.groups) == 2                                  # all keys / a window: own storage
    full = [g for g in cache.groups if g.need.window is None][0]
    assert [tuple(p.shape) for p in full.pools] == [(2, 16, 2, 16, 16)] * 2
    assert cache.view(3).k.data_ptr() == cache.view(0).k.data_ptr() and not cache.view(3).writes
    assert cache.view(2).k.data_ptr() != cache.view(0).k.data_ptr() and cache.view(2).writes
    assert cache.view(1).group != cache.view(0).group
    s = cache.alloc()
    cache.state(1)[s] += 3.0
    cache.reserve(s, 40)
    cache.upload_tables()
    cache.advance(s, 40)
    pages = cache.book.pages[s][0]
    assert cache.groups[0].table[s, :3].tolist() == pages and len(pages) == 3
    assert cache.fits([128] * 1) and not cache.fits([128] * 2)     # 16 pages, 3 in use
    cache.free(s)
    s2 = cache.alloc()
    assert s2 == s and float(cache.state(1)[s2].abs().sum()) == 0  # state zeroed on hand-out
    with pytest.raises(ValueError, match="writes none"):
        SequenceCache({0: CacheNeed(1, 8)}, reads={1: 5}, state_needs={}, max_tokens=64, max_seq=64,
                      dtype=torch.float32, device="cpu")


class _FakeCache:
    def __init__(self, n_slots=4, max_seq=12, capacity=10 ** 9):
        self.free_slots = list(range(n_slots))
        self.max_seq, self.capacity = max_seq, capacity
        self.len = {}
        self.log = []

    def alloc(self):
        s = self.free_slots.pop(0)
        self.len[s] = 0
        self.log.append(("alloc", s))
        return s

    def free(self, s):
        assert s in self.len, "freed twice"
        del self.len[s]
        self.free_slots.append(s)
        self.log.append(("free", s))

    def length(self, s):
        return self.len[s]

    def fits(self, lengths, prompts=None):
        return len(lengths) <= len(self.free_slots) and sum(lengths) <= self.capacity


def _script(cache, script):
    """step_sample that returns, for the sequence in slot s, the next token of script[request]."""
    calls = []
    slot_req = {}

    def step_sample(feed, temps, us):
        calls.append([(s, list(t)) for s, t in feed])
        out = []
        for s, toks in feed:
            if cache.len[s] == 0:
                # identify the request by its prompt
                slot_req[s] = next(r for r, (p, _) in enumerate(script) if list(p) == list(toks))
                step_sample.count[slot_req[s]] = 0
            cache.len[s] += len(toks)
            r = slot_req[s]
            out.append(script[r][1][step_sample.count[r]])
            step_sample.count[r] += 1
        return out
    step_sample.count = {}
    return step_sample, calls


def test_loop_stop_length_and_early_leavers():
    cache = _FakeCache(n_slots=3, max_seq=100)
    script = [([1, 2, 3], [10, 11, 99, 12]),        # stops at 99 after 2 tokens
              ([4], [20, 21, 22, 23, 24]),          # runs to max_tokens = 4
              ([5, 6], [99]),                       # stops at once, emits nothing
              ([7, 8, 9, 9], [30, 31, 32, 33])]     # second batch (only 3 slots)
    fn, calls = _script(cache, script)
    loop = GenerationLoop(fn, cache, max_batch=3)
    res = loop.run([p for p, _ in script], max_tokens=4, temperature=0.0, stop_ids=[99])
    assert [r.tokens for r in res] == [[10, 11], [20, 21, 22, 23], [], [30, 31, 32, 33]]
    assert [r.finish_reason for r in res] == ["stop", "length", "stop", "length"]
    # first batch: prompts of 3 requests in one step, then live ones, one token each
    assert [len(t) for _, t in calls[0]] == [3, 1, 2]
    assert [t for _, t in calls[1]] == [[10], [20]]           # request 2 left after the first step
    assert [t for _, t in calls[2]] == [[11], [21]]
    assert [t for _, t in calls[3]] == [[22]]                 # request 0 left; no step after the last token
    assert len(calls) == 4 + 4
    assert cache.len == {} and sorted(cache.free_slots) == [0, 1, 2]
    allocs = [s for op, s in cache.log if op == "alloc"]
    assert len(allocs) == 4 and len(set(allocs)) == 3          # the second batch uses a slot again
    assert loop.prefill_tokens == 10 and loop.steps == 8


def test_loop_ends_a_sequence_when_its_slot_is_full_and_handles_empty_prompts():
    cache = _FakeCache(n_slots=2, max_seq=6)
    script = [([1, 2, 3, 4], [5, 6, 7, 8, 9]), ([], [])]
    fn, calls = _script(cache, script)
    res = GenerationLoop(fn, cache, 2).run([p for p, _ in script], max_tokens=10)
    # prompt 4 -> sample (len 4), feed -> 5, feed -> 6 = full: the token sampled then cannot be fed
    assert res[0].tokens == [5, 6, 7] and res[0].finish_reason == "length"
    assert res[1].tokens == [] and res[1].finish_reason == "empty"
    assert GenerationLoop(fn, cache, 2).run([[1]], max_tokens=0)[0].finish_reason == "length"
    with pytest.raises(ValueError, match="exceeds the longest"):
        GenerationLoop(fn, cache, 2).run([[1] * 7], max_tokens=1)


def test_loop_batches_by_cache_capacity_and_frees_on_error():
    cache = _FakeCache(n_slots=8, max_seq=50, capacity=30)
    script = [([1] * 5, [2, 2]), ([3] * 6, [4, 4]), ([5] * 20, [6, 6]), ([7] * 2, [8, 8])]
    fn, calls = _script(cache, script)
    GenerationLoop(fn, cache, 8).run([p for p, _ in script], max_tokens=2)
    # 7 + 8 = 15 fit, + 22 = 37 does not: batches are [0, 1], [2, 3]
    assert [len(t) for _, t in calls[0]] == [5, 6] and [len(t) for _, t in calls[2]] == [20, 2]

    def boom(feed, temps, us):
        raise RuntimeError("kernel failed")
    c2 = _FakeCache(n_slots=2)
    with pytest.raises(RuntimeError):
        GenerationLoop(boom, c2, 2).run([[1, 2], [3]], max_tokens=3)
    assert c2.len == {} and len(c2.free_slots) == 2


def test_uniform_depends_on_seed_request_and_step_only():
    a = [uniform(1, r, s) for r in range(4) for s in range(50)]
    assert all(0.0 <= u < 1.0 for u in a) and len(set(a)) == len(a)
    assert a == [uniform(1, r, s) for r in range(4) for s in range(50)]
    assert uniform(2, 0, 0) != uniform(1, 0, 0)
    assert abs(sum(uniform(3, 0, s) for s in range(4000)) / 4000 - 0.5) < 0.03
    assert all(float(torch.tensor(u, dtype=torch.float32)) == u for u in a)   # exact in float32


def test_uniforms_for_a_batch_are_the_single_draws():
    from rbitnet_b200.sampling import uniforms
    for seed in (0, 7, 2 ** 63 + 5, 12345678901234567890):
        reqs, steps = [0, 1, 2, 63, 1000, 2 ** 40], [0, 5, 7, 1023, 99999, 3]
        got = uniforms(seed, reqs, steps)
        assert got.dtype.name == "float32"
        assert got.tolist() == [uniform(seed, r, s) for r, s in zip(reqs, steps)]
    assert uniforms(1, [], []).shape == (0,)


def test_the_decode_step_s_bookkeeping_of_many_slots_is_that_of_one_slot_at_a_time():
    """reserve_one_each / advance_one_each against reserve / advance: same lengths, same pages, same
    rows marked for upload, page after page; and the same error at the end of a sequence's room."""
    def make():
        return SequenceCache({0: CacheNeed(1, 8), 1: CacheNeed(1, 8, window=4)}, reads={}, state_needs={},
                             max_tokens=256, max_seq=40, dtype=torch.float32, device="cpu", page_size=16)
    a, b = make(), make()
    sa, sb = [a.alloc() for _ in range(3)], [b.alloc() for _ in range(3)]
    for c, slots in ((a, sa), (b, sb)):
        for s, n in zip(slots, (1, 15, 16)):
            c.reserve(s, n)
            c.advance(s, n)
    for step in range(24):
        a.reserve_one_each(sa)
        for s in sb:
            b.reserve(s, 1)
        assert a.lengths(sa) == [b.length(s) for s in sb]
        assert [a.book.pages[s] for s in sa] == [b.book.pages[s] for s in sb]
        assert [sorted(g.dirty) for g in a.groups] == [sorted(g.dirty) for g in b.groups]
        a.advance_one_each(sa)
        for s in sb:
            b.advance(s, 1)
        assert a.lengths(sa) == [b.length(s) for s in sb]
    assert a.lengths(sa) == [25, 39, 40]
    with pytest.raises(ContextOverflow):
        a.reserve_one_each(sa)            # the third slot is full


def test_pages_behind_a_window_are_given_back_and_never_a_visible_one():
    """A windowed group holds only the pages its next token can still see; the bound that ``fits`` plans
    with is never exceeded; every page is accounted for at every moment."""
    import random
    rnd = random.Random(5)
    for page, window in [(16, 4), (16, 16), (16, 17), (8, 50), (64, 100)]:
        book = SlotBook(n_slots=3, pages_per_group=[64, 64], page_size=page, max_seq=40 * page,
                        windows=[None, window])
        for trial in range(6):
            s = book.alloc()
            prompt = rnd.randint(1, 6 * page)
            grown = min(book.max_seq, prompt + rnd.randint(0, 10 * page))
            most = [0, 0]
            book.reserve(s, prompt)
            most = [max(m, sum(p >= 0 for p in pg)) for m, pg in zip(most, book.pages[s])]
            book.advance(s, prompt)
            while book.length[s] < grown:
                n = 1 if rnd.random() < 0.8 else min(grown - book.length[s], rnd.randint(1, 2 * page))
                book.reserve(s, n)
                most = [max(m, sum(p >= 0 for p in pg)) for m, pg in zip(most, book.pages[s])]
                # every key the new tokens may see lies on a page the slot still holds
                first_visible = max(0, book.length[s] - window + 1)
                for pos in range(first_visible, book.length[s] + n):
                    assert book.pages[s][1][pos // page] >= 0, (page, window, pos)
                book.advance(s, n)
                for g in (0, 1):
                    held = [p for p in book.pages[s][g] if p >= 0]
                    assert len(held) == len(set(held)) and set(held) <= book.pools[g].held
                    assert book.pools[g].n_free + sum(p >= 0 for p in book.pages[s][g]) == 64
            assert all(p >= 0 for p in book.pages[s][0])                      # the full group keeps everything
            assert most[0] == -(-grown // page)
            assert sum(p >= 0 for p in book.pages[s][1]) <= (window - 1) // page + 2    # what is left at the end
            book.free(s)
            assert all(pool.n_free == 64 for pool in book.pools) and book.slots.n_free == 3
    # the generation loop's case exactly: prompt in one step, then one token at a time
    book = SlotBook(2, [32], 16, 512, windows=[20])
    s = book.alloc()
    book.reserve(s, 100)
    book.advance(s, 100)
    most = sum(p >= 0 for p in book.pages[s][0])
    for _ in range(300):
        book.reserve(s, 1)
        most = max(most, sum(p >= 0 for p in book.pages[s][0]))
        book.advance(s, 1)
    assert most <= book.pages_needed(0, 100, 400) == 7                        # the prompt's 7 pages, then 3 at most
    assert sum(p >= 0 for p in book.pages[s][0]) <= (20 - 1) // 16 + 2


class _FakeDevice:
    """Stands in for an engine whose decode steps leave the next step's tokens on the device: the loop's
    ``step_sample`` (prompts), ``decode_launch`` and ``decode_fetch``.  Every sequence emits its request's
    scripted tokens in order; a launch without tokens feeds what the launch before it sampled, as the
    captured step does."""

    def __init__(self, cache, script):
        self.cache, self.script = cache, script
        self.slot_req, self.count = {}, {}
        self.launches = []            # (slots, tokens fed, had explicit tokens)
        self.results = []
        self.fetched = 0

    def _emit(self, slot):
        r = self.slot_req[slot]
        toks = self.script[r][1]
        i = self.count[r]
        self.count[r] += 1
        return toks[i] if i < len(toks) else -7      # past its script: a sequence that has ended; dropped by the loop

    def step_sample(self, feed, temps, us):
        out = []
        for s, toks in feed:
            assert self.cache.len[s] == 0, "only prompts go through step_sample here"
            self.slot_req[s] = next(r for r, (p, _) in enumerate(self.script) if list(p) == list(toks))
            self.count[self.slot_req[s]] = 0
            self.cache.len[s] += len(toks)
            out.append(self._emit(s))
        return out

    def decode_launch(self, feed, temps, us):
        assert len(self.results) - self.fetched <= 1, "at most two launches are outstanding"
        if feed is not None:
            slots, tokens = [s for s, _ in feed], [t[0] for _, t in feed]
        else:
            slots, tokens = self.launches[-1][0], self.results[-1]
        assert len(temps) == len(us) == len(slots)
        for s in slots:
            if s in self.cache.len:                  # (a slot given back meanwhile is only written to, never read)
                self.cache.len[s] += 1
                assert self.cache.len[s] <= self.cache.max_seq
        self.launches.append((list(slots), list(tokens), feed is not None))
        self.results.append([self._emit(s) for s in slots])
        return len(self.results) - 1

    def decode_fetch(self, ticket):
        assert ticket >= len(self.results) - 2
        self.fetched = max(self.fetched, ticket + 1)
        return self.results[ticket]


@pytest.mark.parametrize("case", range(5))
def test_loop_that_launches_ahead_gives_the_same_results(case):
    """With a decoder the loop launches step k+1 before it reads step k; whatever the scripts (stops at
    any step, several at once, lengths, a full slot), the results are those of the step-by-step loop,
    every token a sequence is fed is the one it sampled before, and no launch follows a known end."""
    scripts = [
        [([1, 2, 3], [10, 11, 99, 12]), ([4], [20, 21, 22, 23, 24, 25, 26]), ([5, 6], [99]),
         ([7, 8, 9, 9], [30, 31, 32, 33, 34, 35, 36])],
        [([1], [5, 5, 5, 99]), ([2], [6, 6, 6, 99]), ([3], [7, 7, 7, 7, 7, 7, 7])],
        [([1, 1], [8] * 9), ([2, 2, 2], [9] * 9)],
        [([1] * 5, [3, 99]), ([2] * 4, [4, 4, 99]), ([3] * 3, [5, 5, 5, 99]), ([4] * 2, [6] * 8)],
        [([1, 2, 3, 4], [5, 6, 7, 8, 9]), ([9], [1, 2, 99])],
    ]
    script = scripts[case]
    max_tokens, max_seq = (6, 100) if case != 4 else (10, 6)
    prompts = [p for p, _ in script]
    seen = {True: [], False: []}
    outs = {}
    for ahead in (False, True):
        cache = _FakeCache(n_slots=3, max_seq=max_seq)
        dev = _FakeDevice(cache, script)
        loop = GenerationLoop(dev.step_sample if ahead else _script(cache, script)[0], cache, 3,
                              decoder=dev if ahead else None)
        outs[ahead] = loop.run(prompts, max_tokens=max_tokens, stop_ids=[99],
                               on_token=lambda r, t, a=ahead: seen[a].append((r, t)))
        assert cache.len == {} and sorted(cache.free_slots) == [0, 1, 2]
        if ahead:
            assert any(not explicit for _, _, explicit in dev.launches) or case == 4 or max(len(t) for _, t in script) < 3
            for (slots, tokens, explicit), prev in zip(dev.launches[1:], dev.launches[:-1]):
                if not explicit:
                    assert slots == prev[0]                       # the same sequences, their tokens from the device
            # every explicitly fed token is the last one its sequence emitted
            for slots, tokens, explicit in dev.launches:
                if explicit:
                    for s_, t_ in zip(slots, tokens):
                        assert t_ != 99 and t_ != -7
    got = [(r.tokens, r.finish_reason, r.prompt_tokens) for r in outs[True]]
    assert got == [(r.tokens, r.finish_reason, r.prompt_tokens) for r in outs[False]]
    assert sorted(seen[True]) == sorted(seen[False])
    for r in range(len(script)):                                  # per request the tokens come in order
        assert [t for q, t in seen[True] if q == r] == outs[True][r].tokens
