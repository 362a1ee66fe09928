"""Each kernel alone against a plain torch float32 reference of the same operation, at sizes
other than the engine's test models: widths and vocabularies that are no power of two, head sizes
in steps of 16, odd head counts and groups, token counts that do not fill a tile."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16, F32 = torch.bfloat16, torch.float32


@pytest.fixture(scope="module")
def ops32():
    from rbitnet_b200.kernels.ops import CudaOps
    return CudaOps(F32)


@pytest.fixture(scope="module")
def ops16():
    from rbitnet_b200.kernels.ops import CudaOps
    return CudaOps(BF16)


def _rel(got, ref):
    return float((got.double() - ref.double()).abs().max()) / max(float(ref.double().abs().max()), 1e-30)


def test_extension_is_loaded_from_the_tree(ops16):
    import os
    assert "librbitnet_b200_" in ops16.lib.path and os.path.isfile(ops16.lib.path)
    maps = open("/proc/self/maps").read()
    assert os.path.basename(ops16.lib.path) in maps


@pytest.mark.parametrize("V,E,T", [(257, 48, 5), (1000, 272, 33), (300, 4100, 7), (100, 50, 3), (64, 2049, 2)])
def test_embed(ops32, ops16, V, E, T):
    g = torch.Generator(device="cuda").manual_seed(1)
    table = torch.randn(V, E, device="cuda", generator=g)
    ids = torch.randint(0, V, (T,), device="cuda", generator=g, dtype=torch.int32)
    assert torch.equal(ops32.embed(ids, table), table[ids.long()])
    tb = table.to(BF16)
    assert torch.equal(ops16.embed(ids, tb), tb[ids.long()].float())


@pytest.mark.parametrize("E,T,eps", [(48, 3, 1e-5), (272, 17, 1e-6), (4096, 5, 1e-5), (5000, 2, 1e-3), (50, 3, 1e-5), (18000, 2, 1e-5)])
def test_rmsnorm(ops32, ops16, E, T, eps):
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(T, E, device="cuda", generator=g) * 3
    w = 1 + 0.1 * torch.randn(E, device="cuda", generator=g)
    ref = (x.double() * w.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps))
    assert _rel(ops32.rmsnorm(x.clone(), w, eps), ref) < 2e-6
    assert _rel(ops16.rmsnorm(x.clone(), w, eps), ref) < 5e-3


@pytest.mark.parametrize("T,N,K", [(1, 7, 5), (3, 100, 33), (70, 130, 257), (5, 48, 176)])
def test_plain_product_is_true_float32(ops32, T, N, K):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(T, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g)
    ref = x.double() @ w.double().T
    got = ops32.linear(x, ops32.prepare_linear([w]))
    assert _rel(got, ref) < 1e-6        # a reduced-precision matrix mode would give ~1e-3
    acc = torch.randn(T, N, device="cuda", generator=g)
    want = acc.double() + ref
    ops32.linear(x, ops32.prepare_linear([w]), accumulate_into=acc)
    assert _rel(acc, want) < 1e-6


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (5, 200, 96), (17, 1000, 176), (64, 384, 520), (100, 130, 4096),
                                   (129, 257, 72), (300, 520, 1032), (700, 96, 48),
                                   # 65 to 256 tokens: token tiles of 64, several of them, with K cut or not
                                   (130, 4096, 4096), (200, 1000, 14336), (256, 6144, 1024), (250, 28000, 512),
                                   # 257 to 1024 tokens: tiles of 128 or 256, whichever needs fewer rounds of the SMs
                                   (500, 4096, 1032), (512, 28672, 256), (1000, 6144, 512), (1024, 4096, 520)])
def test_tensor_core_product(ops16, T, N, K):
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(T, K, device="cuda", generator=g).to(BF16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(BF16)
    ref = x.double() @ w.double().T
    lw = ops16.prepare_linear([w])
    assert ops16._tensor_core_ok(x, lw.w)
    assert _rel(ops16.linear(x, lw, out_dtype=F32), ref) < 2e-5          # float32 accumulation
    assert _rel(ops16.linear(x, lw), ref) < 5e-3                          # rounded to bfloat16 once
    acc = torch.randn(T, N, device="cuda", generator=g)
    want = acc.double() + ref
    ops16.linear(x, lw, accumulate_into=acc)
    assert _rel(acc, want) < 2e-5
    ops16.check_errors()


@pytest.mark.parametrize("T", [1, 8, 64, 2048])
def test_products_at_the_layer_sizes_of_llama_3_8b(ops16, T):
    """The products of one layer and the head at hidden 4096, inner 14336, vocabulary 128256: more
    tiles than CTAs run at once (each CTA takes several, its two accumulators in turn), K cut into
    clusters for few tokens, the widest token tile for many."""
    g = torch.Generator(device="cuda").manual_seed(40 + T)
    E, F, V, QKV = 4096, 14336, 128256, 6144
    x = torch.randn(T, E, device="cuda", generator=g).to(BF16)

    def weight(n, k):
        return (torch.randn(n, k, device="cuda", generator=g) / math.sqrt(k)).to(BF16)

    def ref(a, w):
        return a.double() @ w.double().T

    w = weight(QKV, E)
    assert _rel(ops16.linear(x, ops16.prepare_linear([w])), ref(x, w)) < 5e-3
    w = weight(E, E)
    acc = torch.randn(T, E, device="cuda", generator=g)
    want = acc.double() + ref(x, w)
    ops16.linear(x, ops16.prepare_linear([w]), accumulate_into=acc)
    assert _rel(acc, want) < 2e-5
    wg, wu = weight(F, E) * 2, weight(F, E)
    gate, up = ref(x, wg), ref(x, wu)
    t = ops16.gated_linear(x, ops16.prepare_gate_up(wg, wu))
    assert _rel(t, gate / (1 + torch.exp(-gate)) * up) < 6e-3
    del wg, wu, gate, up
    w = weight(E, F)
    acc = torch.randn(T, E, device="cuda", generator=g)
    want = acc.double() + ref(t, w)
    ops16.linear(t, ops16.prepare_linear([w]), accumulate_into=acc)
    assert _rel(acc, want) < 2e-5
    del w
    rows = x[:min(T, 64)].contiguous()                     # the head sees the wanted rows only
    w = weight(V, E)
    assert _rel(ops16.linear(rows, ops16.prepare_linear([w]), out_dtype=F32), ref(rows, w)) < 2e-5
    ops16.check_errors()


def test_product_refuses_to_guess_for_odd_inner_sizes(ops16):
    """An inner size TMA cannot address goes to the plain product, with the same result."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(9, 77, device="cuda", generator=g).to(BF16)
    w = torch.randn(50, 77, device="cuda", generator=g).to(BF16)
    lw = ops16.prepare_linear([w])
    assert not ops16._tensor_core_ok(x, lw.w)
    assert _rel(ops16.linear(x, lw, out_dtype=F32), x.double() @ w.double().T) < 2e-5
    from rbitnet_b200.kernels.lib import KernelError
    with pytest.raises(KernelError, match="multiple of 8"):
        ops16.lib.call("rb_gemm_tc", 0, 50, 1, 0, 77, 9, 0, 77, 50, 50, 77, 0, 0, 1, 0, 1.0, 0)


@pytest.mark.parametrize("T,F,K", [(1, 176, 64), (40, 352, 96), (130, 1000, 256), (300, 129, 72)])
def test_gated_feed_forward_product(ops32, ops16, T, F, K):
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(T, K, device="cuda", generator=g)
    wg = torch.randn(F, K, device="cuda", generator=g) / math.sqrt(K) * 2
    wu = torch.randn(F, K, device="cuda", generator=g) / math.sqrt(K)
    for ops, tol in ((ops32, 2e-6), (ops16, 6e-3)):
        xx, g_, u_ = (t.to(ops.dtype) for t in (x, wg, wu))
        gate, up = xx.double() @ g_.double().T, xx.double() @ u_.double().T
        ref = gate / (1 + torch.exp(-gate)) * up
        got = ops.gated_linear(xx, ops.prepare_gate_up(g_, u_))
        assert got.shape == (T, F) and _rel(got, ref) < tol


class _Meta:
    pass


def _paged(ops, n_slots, max_pages, page, Kh, D, lens, seed):
    """A cache with shuffled pages, filled with random keys and values for sequences of ``lens``."""
    from rbitnet_b200.cache import CacheLayerView
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_pages = n_slots * max_pages
    # places no sequence owns hold large values: a key read past a sequence's end would show
    k = (torch.randn(n_pages, Kh, page, D, device="cuda", generator=g) * 30).to(ops.dtype)
    v = (torch.randn(n_pages, Kh, page, D, device="cuda", generator=g) * 30).to(ops.dtype)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    table_host = perm.reshape(n_slots, max_pages)
    table = table_host.cuda()
    dense_k, dense_v = [], []
    for s, n in enumerate(lens):
        kk = torch.randn(n, Kh, D, device="cuda", generator=g).to(ops.dtype)
        vv = torch.randn(n, Kh, D, device="cuda", generator=g).to(ops.dtype)
        for p0 in range(0, n, page):
            pg, m = int(table_host[s, p0 // page]), min(page, n - p0)
            k[pg, :, :m] = kk[p0:p0 + m].transpose(0, 1)
            v[pg, :, :m] = vv[p0:p0 + m].transpose(0, 1)
        dense_k.append(kk)
        dense_v.append(vv)
    return CacheLayerView(k, v, table, max_pages, page, Kh, D, True, 0), dense_k, dense_v


def _attn_ref(q, k, v, pos, scale, window):
    """q [H, D] at position pos over k, v [n, Kh, D], float64."""
    H, D = q.shape
    G = H // k.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    out = torch.zeros(H, D, dtype=torch.float64, device=q.device)
    for h in range(H):
        s = (k[lo:pos + 1, h // G].double() @ q[h].double()) * scale
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, h // G].double()
    return out.reshape(-1)


def _meta(rows, single_token=False, max_context=512):
    """rows: (slot, position) per batch row; consecutive positions of one slot form one chunk."""
    from rbitnet_b200.engine.step import SeqChunk
    m = _Meta()
    m.tok_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32, device="cuda")
    m.tok_pos = torch.tensor([r[1] for r in rows], dtype=torch.int32, device="cuda")
    m.seqs, i = [], 0
    while i < len(rows):
        j = i + 1
        while j < len(rows) and rows[j][0] == rows[i][0] and rows[j][1] == rows[j - 1][1] + 1:
            j += 1
        m.seqs.append(SeqChunk(rows[i][0], rows[i][1], j - i, i))
        i = j
    m.single_token, m.max_context, m.extra = single_token, max_context, {}
    m.n_tokens = len(rows)
    return m


ATTN_CASES = [(4, 2, 16, 16, None), (3, 1, 32, 64, None), (6, 3, 48, 16, 5), (8, 2, 128, 64, None),
              (5, 5, 80, 32, 40), (2, 1, 256, 16, None), (6, 2, 64, 64, 100), (32, 8, 128, 128, None),
              (7, 7, 96, 64, None), (4, 1, 112, 64, 33), (18, 1, 16, 64, None), (2, 2, 256, 64, None),
              (16, 1, 128, 64, 70), (12, 4, 64, 128, None)]


@pytest.mark.parametrize("H,Kh,D,page,window", ATTN_CASES)
def test_attention_over_the_paged_cache(ops32, ops16, H, Kh, D, page, window):
    """Queries at mixed positions of three sequences: runs of prompt rows (long enough to cross
    tiles and the diagonal) and single rows in one batch."""
    lens = [200, 9, 130]
    scale = 0.7 / math.sqrt(D)
    max_pages = -(-256 // page)
    for ops, tol in ((ops32, 3e-6), (ops16, 8e-3)):
        view, ks, vs = _paged(ops, 3, max_pages, page, Kh, D, lens, seed=7)
        rows = ([(0, 69), (1, 0), (1, 8), (2, 64), (2, 129), (0, 5)] + [(2, p) for p in range(100, 110)]
                + [(0, p) for p in range(30, 200)] + [(1, p) for p in range(0, 9)])
        g = torch.Generator(device="cuda").manual_seed(8)
        q = torch.randn(len(rows), H, D, device="cuda", generator=g).to(ops.dtype) * 2
        got = ops.attention(q, _meta(rows), view, H, scale, window)
        for i, (s, p) in enumerate(rows):
            if i > 20 and i % 7:
                continue
            ref = _attn_ref(q[i], ks[s], vs[s], p, scale, window)
            assert _rel(got[i], ref) < tol, (i, s, p)


@pytest.mark.parametrize("H,Kh,D,page,window", ATTN_CASES)
@pytest.mark.parametrize("max_context", [64, 128, 256, 700, 1100])
def test_decode_attention_with_split_keys(ops16, H, Kh, D, page, window, max_context):
    """One token per sequence at the end of sequences of very different lengths; the keys are cut
    into parts (how many depends on the batch and on max_context: here 1, 2, 4, 8 and 16 for the
    TMA-fed kernel, some of them without keys) and merged, inside a thread-block cluster or by a
    second kernel."""
    lens = [1, 700, 64, 65, 333]
    scale = 1.3 / math.sqrt(D)
    view, ks, vs = _paged(ops16, len(lens), -(-704 // page), page, Kh, D, lens, seed=12)
    rows = [(s, n - 1) for s, n in enumerate(lens)]
    g = torch.Generator(device="cuda").manual_seed(13)
    q = torch.randn(len(rows), H, D, device="cuda", generator=g).to(BF16) * 2
    got = ops16.attention(q, _meta(rows, single_token=True, max_context=max_context), view, H, scale, window)
    for i, (s, p) in enumerate(rows):
        assert _rel(got[i], _attn_ref(q[i], ks[s], vs[s], p, scale, window)) < 8e-3, (i, s, p)


@pytest.mark.parametrize("H,Kh,D", [(8, 4, 64), (8, 4, 128)])
def test_decode_attention_of_many_sequences(ops16, H, Kh, D):
    """More (sequence, kv head) pairs than run at once: the keys are then cut into a number of parts
    that fills whole waves, and a second kernel merges them."""
    lens = [1 + (37 * i) % 250 for i in range(150)]
    scale = 1.1 / math.sqrt(D)
    view, ks, vs = _paged(ops16, len(lens), 4, 64, Kh, D, lens, seed=21)
    rows = [(s, n - 1) for s, n in enumerate(lens)]
    parts = ops16.lib.raw("rb_attention_decode_tma_parts")(len(rows) * Kh, 4, D)
    assert parts > 1 and not ops16.lib.raw("rb_attention_decode_tma_on_chip")(len(rows) * Kh, parts, D)
    g = torch.Generator(device="cuda").manual_seed(22)
    q = torch.randn(len(rows), H, D, device="cuda", generator=g).to(BF16) * 2
    got = ops16.attention(q, _meta(rows, single_token=True, max_context=250), view, H, scale, None)
    for i, (s, p) in enumerate(rows):
        if i % 5 == 0 or p < 3:
            assert _rel(got[i], _attn_ref(q[i], ks[s], vs[s], p, scale, None)) < 8e-3, (i, s, p)


@pytest.mark.parametrize("window", [None, 1000])
def test_attention_at_a_context_of_2100(ops16, window):
    """Heads as in Llama-3-8B, a sequence of 2,100 positions beside a short one: its whole prompt in
    one step (17 key tiles of 128 for the last rows), then one token each (33 tiles of 64 cut into
    16 parts)."""
    H, Kh, D, page = 32, 8, 128, 64
    lens = [2100, 300]
    scale = 1.0 / math.sqrt(D)
    view, ks, vs = _paged(ops16, 2, -(-2112 // page), page, Kh, D, lens, seed=31)
    rows = [(0, p) for p in range(2100)] + [(1, p) for p in range(300)]
    g = torch.Generator(device="cuda").manual_seed(32)
    q = torch.randn(len(rows), H, D, device="cuda", generator=g).to(BF16) * 2
    got = ops16.attention(q, _meta(rows, max_context=2100), view, H, scale, window)
    for i in [0, 63, 64, 127, 128, 999, 1000, 1001, 2047, 2048, 2099, 2100, 2399]:
        s, p = rows[i]
        assert _rel(got[i], _attn_ref(q[i], ks[s], vs[s], p, scale, window)) < 8e-3, (i, s, p)
    last = [(0, 2099), (1, 299)]
    q1 = torch.randn(2, H, D, device="cuda", generator=g).to(BF16) * 2
    got = ops16.attention(q1, _meta(last, single_token=True, max_context=2100), view, H, scale, window)
    for i, (s, p) in enumerate(last):
        assert _rel(got[i], _attn_ref(q1[i], ks[s], vs[s], p, scale, window)) < 8e-3, (i, s, p)
    ops16.check_errors()


def test_attention_finds_one_far_key_and_respects_the_window_edge(ops32):
    """One key matches the query strongly.  Inside the mask it must dominate the output; one
    position outside the window it must not be seen at all."""
    H, Kh, D, page, n = 2, 1, 32, 16, 300
    view, ks, vs = _paged(ops32, 1, 32, page, Kh, D, [n], seed=9)
    q = torch.zeros(1, H, D, device="cuda")
    q[0, :, 3] = 50.0
    far = 17
    for kk in (ks[0],):
        kk[:, :, 3] = 0.0
        kk[far, 0, 3] = 10.0
    pg = int(view.page_table[0, far // page])
    view.k[:, :, :, 3] = 0.0
    view.k[pg, 0, far % page, 3] = 10.0
    meta = _meta([(0, n - 1)])
    scale = 1 / math.sqrt(D)
    out = ops32.attention(q, meta, view, H, scale, None).reshape(H, D)
    assert _rel(out[0], vs[0][far, 0]) < 1e-5                       # the far key owns the softmax
    w_in, w_out = n - far, n - far - 1                               # window that just reaches it / just misses
    assert _rel(ops32.attention(q, meta, view, H, scale, w_in).reshape(H, D)[0], vs[0][far, 0]) < 1e-5
    missed = ops32.attention(q, meta, view, H, scale, w_out).reshape(H, D)[0]
    ref = vs[0][far + 1:n, 0].double().mean(0)                       # all other scores are equal (zero)
    assert _rel(missed, ref) < 1e-5


@pytest.mark.parametrize("H,Kh,D,interleaved", [(4, 2, 16, True), (3, 1, 32, False), (8, 8, 64, False), (2, 1, 128, True)])
def test_rotation_and_cache_append(ops32, ops16, H, Kh, D, interleaved):
    from rbitnet_b200.cache import CacheLayerView
    theta = 10000.0 if interleaved else 500000.0
    page, max_pages, n_slots = 16, 8, 3
    rows = [(0, 0), (0, 1), (2, 100), (1, 15), (1, 16), (2, 127)]
    T = len(rows)
    for ops, tol in ((ops32, 2e-6), (ops16, 6e-3)):
        g = torch.Generator(device="cuda").manual_seed(10)
        qkv = torch.randn(T, (H + 2 * Kh) * D, device="cuda", generator=g).to(ops.dtype)
        k = torch.zeros(n_slots * max_pages, Kh, page, D, device="cuda", dtype=ops.dtype)
        v = torch.zeros_like(k)
        table = torch.randperm(n_slots * max_pages).to(torch.int32).reshape(n_slots, max_pages).cuda()
        view = CacheLayerView(k, v, table, max_pages, page, Kh, D, True, 0)
        meta = _meta(rows)
        i = torch.arange(D // 2, dtype=torch.float32)
        inv = (1.0 / torch.pow(torch.tensor(theta), 2.0 * i / D)).cuda()
        q = ops.rotate_append(qkv, (inv, interleaved, D), meta, view, H)

        def rot(x, pos):     # x [heads, D] float64
            ang = (torch.tensor(float(pos), dtype=torch.float32) * inv.cpu()).double()
            c, s = torch.cos(ang), torch.sin(ang)
            out = torch.empty_like(x)
            if interleaved:
                a, b = x[:, 0::2], x[:, 1::2]
                out[:, 0::2], out[:, 1::2] = a * c - b * s, a * s + b * c
            else:
                a, b = x[:, :D // 2], x[:, D // 2:]
                out[:, :D // 2], out[:, D // 2:] = a * c - b * s, a * s + b * c
            return out

        x = qkv.double().cpu()
        for t, (slot, pos) in enumerate(rows):
            assert _rel(q[t].cpu(), rot(x[t, :H * D].reshape(H, D), pos)) < tol
            pg = int(table[slot, pos // page])
            assert _rel(k[pg, :, pos % page].cpu(), rot(x[t, H * D:(H + Kh) * D].reshape(Kh, D), pos)) < tol
            assert torch.equal(v[pg, :, pos % page].cpu().double(), x[t, (H + Kh) * D:].reshape(Kh, D))
        written = sum(1 for _ in rows)
        assert int((k.abs().sum(dim=(1, 3)) > 0).sum()) == written       # nothing else was touched


@pytest.mark.parametrize("H,Kh,D,interleaved,K,T,writes", [
    (4, 2, 16, True, 512, 5, True), (3, 1, 32, False, 1024, 6, True), (8, 8, 64, False, 2048, 1, True),
    (6, 2, 128, True, 4096, 6, True), (5, 1, 64, False, 1024, 6, False), (2, 1, 128, False, 520, 40, True)])
@pytest.mark.parametrize("pending", [False, True])
def test_qkv_product_that_rotates_and_appends_in_its_epilogue(ops16, H, Kh, D, interleaved, K, T, writes, pending):
    """The q/k/v product of a few tokens whose epilogue rotates q and k and writes k and v into the paged
    cache, against the product in float64 followed by the rotation; and the step's own choice of path.
    ``pending``: the input rows come with their norm pending (rows times the norm's weights, and sums of
    squares in three parts), and the product multiplies its sums by each row's factor."""
    from rbitnet_b200.cache import CacheLayerView
    from rbitnet_b200.kernels.ops import NormedRows
    theta = 10000.0 if interleaved else 500000.0
    page, max_pages, n_slots = 16, 8, 6
    places = [(0, 0), (0, 1), (2, 100), (1, 15), (1, 16), (2, 127)]
    rows = [places[i % 6] if i < 6 else (3 + (i - 6) // 20, i) for i in range(T)]
    g = torch.Generator(device="cuda").manual_seed(31)
    n_out = (H + (2 * Kh if writes else 0)) * D
    h = torch.randn(T, K, device="cuda", generator=g).to(BF16)
    w = (torch.randn(n_out, K, device="cuda", generator=g) / math.sqrt(K)).to(BF16)
    lw = ops16.prepare_linear([w])
    k = torch.zeros(n_slots * max_pages, Kh, page, D, device="cuda", dtype=BF16)
    v = torch.zeros_like(k)
    table = torch.randperm(n_slots * max_pages).to(torch.int32).reshape(n_slots, max_pages).cuda()
    view = CacheLayerView(k, v, table, max_pages, page, Kh, D, writes, 0)
    meta = _meta(rows)
    i = torch.arange(D // 2, dtype=torch.float32)
    inv = (1.0 / torch.pow(torch.tensor(theta), 2.0 * i / D)).cuda()
    splits = ops16._k_splits(T, n_out, K)
    fused = bool(ops16.lib.raw("rb_gemm_tc_qkv_supports")(T, D, splits))
    assert fused == (splits >= 2 and T <= 16), (splits, fused)
    given = h
    if pending:
        rows_f = torch.randn(T, K, device="cuda", generator=g) * 3.0
        gw = 1.0 + 0.5 * torch.randn(K, device="cuda", generator=g)
        eps = 1e-5
        scaled = (rows_f * gw).to(BF16)
        cut = torch.rand(3, T, device="cuda", generator=g)
        squares = (cut / cut.sum(0)) * (rows_f * rows_f).sum(-1)
        given = NormedRows(rows_f, gw, eps, scaled, squares.contiguous())
        factor = 1.0 / torch.sqrt((rows_f.double() ** 2).mean(-1) + eps)
        h = scaled.double() * factor[:, None]                # what the product should see, in float64
    before = ops16.lib.launches
    q = ops16.project_rotate_append(given, lw, (inv, interleaved, D), meta, view, H)
    # (rows with a pending norm are taken as they are up to 16 tokens; beyond, the norm's own kernel runs first)
    assert ops16.lib.launches - before == (1 if fused else 2) + (1 if pending and T > 16 else 0)
    ops16.check_errors()

    def rot(x, pos):     # x [heads, D] float64
        ang = (torch.tensor(float(pos), dtype=torch.float32) * inv.cpu()).double()
        c, s = torch.cos(ang), torch.sin(ang)
        out = torch.empty_like(x)
        if interleaved:
            a, b = x[:, 0::2], x[:, 1::2]
            out[:, 0::2], out[:, 1::2] = a * c - b * s, a * s + b * c
        else:
            a, b = x[:, :D // 2], x[:, D // 2:]
            out[:, :D // 2], out[:, D // 2:] = a * c - b * s, a * s + b * c
        return out

    x = (h.double() @ w.double().T).cpu()
    scale = float(x.abs().max())
    for t, (slot, pos) in enumerate(rows):
        assert float((q[t].cpu().double() - rot(x[t, :H * D].reshape(H, D), pos)).abs().max()) < 6e-3 * scale
        if writes:
            pg = int(table[slot, pos // page])
            got_k, got_v = k[pg, :, pos % page].cpu().double(), v[pg, :, pos % page].cpu().double()
            assert float((got_k - rot(x[t, H * D:(H + Kh) * D].reshape(Kh, D), pos)).abs().max()) < 6e-3 * scale
            assert float((got_v - x[t, (H + Kh) * D:].reshape(Kh, D)).abs().max()) < 6e-3 * scale
    if writes:
        assert int((k.abs().sum(dim=(1, 3)) > 0).sum()) == len(set(rows))       # nothing else was touched
    else:
        assert float(k.abs().sum()) == 0 and float(v.abs().sum()) == 0


@pytest.mark.parametrize("V", [257, 1000, 128256])
def test_sampling(ops32, V):
    import plain_llama as plain
    g = torch.Generator(device="cuda").manual_seed(11)
    R = 6
    logits = torch.randn(R, V, device="cuda", generator=g) * 3
    logits[1, 5] = float("nan")
    logits[2, 40] = logits[2, 41] = 99.0                       # a tie: the lowest index wins
    logits[3] = float("nan")
    logits[3, 7] = -2.0
    zero = torch.zeros(R, device="cuda")
    got = ops32.sample(logits, zero, zero).tolist()
    for r in range(R):
        assert got[r] == plain.greedy_token(logits[r].cpu())
    assert got[2] == 40 and got[3] == 7
    temps = torch.tensor([0.5, 1.0, 0.8, 1.0, 2.0, 0.0], device="cuda")
    for trial in range(5):
        u = torch.rand(R, generator=torch.Generator().manual_seed(trial)).cuda()
        got = ops32.sample(logits, temps, u).tolist()
        for r in range(R - 1):
            cdf = plain.temperature_cdf(torch.nan_to_num(logits[r].cpu(), nan=-float("inf")), float(temps[r]))
            total, target = float(cdf[-1]), float(u[r]) * float(cdf[-1])
            i = got[r]
            below = float(cdf[i - 1]) if i > 0 else 0.0
            assert below - 1e-5 * total <= target <= float(cdf[i]) + 1e-5 * total, (r, i)
        assert got[R - 1] == plain.greedy_token(logits[R - 1].cpu())
    # the edges of the unit interval
    flat = torch.zeros(2, V, device="cuda")
    one = torch.ones(2, device="cuda")
    assert ops32.sample(flat, one, torch.tensor([0.0, 0.99999994], device="cuda")).tolist() == [0, V - 1]


@pytest.mark.parametrize("E", [48, 50, 1028, 3001])
def test_gather_rows(ops32, E):
    x = torch.randn(20, E, device="cuda")
    rows = torch.tensor([19, 0, 7, 7], dtype=torch.int32, device="cuda")
    assert torch.equal(ops32.gather_rows(x, rows), x[rows.long()])


@pytest.mark.parametrize("T,N,K", [(1, 256, 4096), (8, 100, 1032), (64, 4096, 1024), (33, 520, 2048), (5, 6144, 4096)])
def test_product_split_along_the_inner_dimension(ops16, T, N, K):
    """Few tokens and few weight tiles: the inner dimension is cut into parts whose CTAs form a
    cluster; the first of them adds the parts up on chip, in a fixed order."""
    g = torch.Generator(device="cuda").manual_seed(14)
    x = torch.randn(T, K, device="cuda", generator=g).to(BF16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(BF16)
    lw = ops16.prepare_linear([w])
    assert 1 < ops16._k_splits(T, N, K) <= 8
    ref = x.double() @ w.double().T
    y = ops16.linear(x, lw, out_dtype=F32)
    assert _rel(y, ref) < 2e-5
    assert torch.equal(y, ops16.linear(x, lw, out_dtype=F32))          # the same bits every time
    assert _rel(ops16.linear(x, lw), ref) < 5e-3
    acc = torch.randn(T, N, device="cuda", generator=g)
    want = acc.double() + ref
    ops16.linear(x, lw, accumulate_into=acc)
    assert _rel(acc, want) < 2e-5
    ops16.check_errors()


@pytest.mark.parametrize("H,Kh,D,interleaved", [(4, 2, 16, True), (3, 1, 48, False), (8, 2, 128, False), (2, 2, 256, True)])
def test_rotation_of_many_tokens(ops16, H, Kh, D, interleaved):
    """The many-token form of the rotation (one block per token, 16-byte accesses) against the
    few-token form on the same rows."""
    from rbitnet_b200.cache import CacheLayerView
    page, max_pages, n_slots, T = 64, 4, 2, 200
    rows = [(0, p) for p in range(130)] + [(1, p) for p in range(17, 17 + T - 130)]
    g = torch.Generator(device="cuda").manual_seed(16)
    qkv = torch.randn(T, (H + 2 * Kh) * D, device="cuda", generator=g).to(BF16)
    inv = (1.0 / torch.pow(torch.tensor(10000.0), 2.0 * torch.arange(D // 2, dtype=torch.float32) / D)).cuda()
    table = torch.randperm(n_slots * max_pages).to(torch.int32).reshape(n_slots, max_pages).cuda()
    res = []
    for chunk in (T, 100):      # 200 rows at once (many-token kernel), or in two steps of 100 (few-token kernel)
        k = torch.zeros(n_slots * max_pages, Kh, page, D, device="cuda", dtype=BF16)
        v = torch.zeros_like(k)
        view = CacheLayerView(k, v, table, max_pages, page, Kh, D, True, 0)
        qs = [ops16.rotate_append(qkv[i:i + chunk], (inv, interleaved, D), _meta(rows[i:i + chunk]), view, H)
              for i in range(0, T, chunk)]
        res.append((torch.cat(qs), k, v))
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a, b)


# --------------------------------------------------------------------------- further sizes and options
@pytest.mark.parametrize("n_seqs", [64, 1])
def test_decode_attention_at_8192_positions(ops16, n_seqs):
    """Heads as in Llama-3-8B at 8,192 cached positions.  64 sequences: more CTAs than run at once, any
    number of parts up to 16, merged by the second kernel.  One sequence: sixteen parts, one
    thread-block cluster that merges on chip."""
    H, Kh, D, page = 32, 8, 128, 64
    top = 8192
    lens = [top] if n_seqs == 1 else [top - (i * 997) % 6000 for i in range(n_seqs)]
    lens[0] = top
    scale = 1.0 / math.sqrt(D)
    view, ks, vs = _paged(ops16, n_seqs, top // page, page, Kh, D, lens, seed=61)
    rows = [(s, n - 1) for s, n in enumerate(lens)]
    parts = ops16.lib.raw("rb_attention_decode_tma_parts")(n_seqs * Kh, top // 64, D)
    on_chip = bool(ops16.lib.raw("rb_attention_decode_tma_on_chip")(n_seqs * Kh, parts, D))
    assert parts > 1 and on_chip == (n_seqs == 1)
    g = torch.Generator(device="cuda").manual_seed(62)
    q = torch.randn(n_seqs, H, D, device="cuda", generator=g).to(BF16) * 2
    got = ops16.attention(q, _meta(rows, single_token=True, max_context=top), view, H, scale, None)
    ops16.check_errors()
    for i in sorted({0, min(1, n_seqs - 1), n_seqs // 2, n_seqs - 1}):
        s, p = rows[i]
        assert _rel(got[i], _attn_ref(q[i], ks[s], vs[s], p, scale, None)) < 8e-3, (i, s, p)
    # one key far back carries the answer: its score is made to stand out, its value is marked
    far = 100
    pg = int(view.page_table[0, far // page])
    kq = view.k[pg, :, far % page].float()                          # [Kh, D]
    q2 = q.clone()
    q2[0] = (kq.repeat_interleave(H // Kh, dim=0) * 4).to(BF16)     # q . k_far is far above every other score
    got = ops16.attention(q2, _meta(rows, single_token=True, max_context=top), view, H, scale, None)
    want = view.v[pg, :, far % page].float().repeat_interleave(H // Kh, dim=0).reshape(-1)
    assert _rel(got[0], want.double()) < 2e-2


@pytest.mark.parametrize("H,Kh,D,rot,interleaved", [(4, 2, 16, 8, True), (3, 1, 32, 16, False), (8, 2, 128, 64, False),
                                                    (2, 1, 64, 0, True), (2, 2, 128, 32, True)])
def test_rotation_of_a_prefix_of_each_head(ops32, ops16, H, Kh, D, rot, interleaved):
    """Only the first ``rot`` values of a head are rotated (pairs among them), the rest pass as they
    are: by the rotation kernel (few and many tokens) and by the q/k/v product's epilogue."""
    from rbitnet_b200.cache import CacheLayerView
    page, max_pages, n_slots = 16, 8, 4
    i = torch.arange(max(rot // 2, 1), dtype=torch.float32)
    inv = (1.0 / torch.pow(torch.tensor(10000.0), 2.0 * i / max(rot, 2))).cuda()

    def rotated(x, pos):     # x [heads, D] float64
        out = x.clone()
        if rot == 0:
            return out
        ang = (torch.tensor(float(pos), dtype=torch.float32) * inv.cpu()[:rot // 2]).double()
        c, s = torch.cos(ang), torch.sin(ang)
        if interleaved:
            a, b = x[:, 0:rot:2], x[:, 1:rot:2]
            out[:, 0:rot:2], out[:, 1:rot:2] = a * c - b * s, a * s + b * c
        else:
            a, b = x[:, :rot // 2], x[:, rot // 2:rot]
            out[:, :rot // 2], out[:, rot // 2:rot] = a * c - b * s, a * s + b * c
        return out

    def check(ops, tol, T, through_product):
        rows = [(t % n_slots, (7 * t) % 120) for t in range(T)]
        rows = sorted(set(rows))[:T]
        T = len(rows)
        g = torch.Generator(device="cuda").manual_seed(70 + T)
        k = torch.zeros(n_slots * max_pages, Kh, page, D, device="cuda", dtype=ops.dtype)
        v = torch.zeros_like(k)
        table = torch.randperm(n_slots * max_pages).to(torch.int32).reshape(n_slots, max_pages).cuda()
        view = CacheLayerView(k, v, table, max_pages, page, Kh, D, True, 0)
        n_out = (H + 2 * Kh) * D
        if through_product:
            K = 1024
            h = torch.randn(T, K, device="cuda", generator=g).to(ops.dtype)
            w = (torch.randn(n_out, K, device="cuda", generator=g) / math.sqrt(K)).to(ops.dtype)
            before = ops.lib.launches
            q = ops.project_rotate_append(h, ops.prepare_linear([w]), (inv, interleaved, rot), _meta(rows), view, H)
            assert ops.lib.launches - before == 1                  # the product's own epilogue did it
            x = (h.double() @ w.double().T).cpu()
        else:
            qkv = torch.randn(T, n_out, device="cuda", generator=g).to(ops.dtype)
            q = ops.rotate_append(qkv, (inv, interleaved, rot), _meta(rows), view, H)
            x = qkv.double().cpu()
        scale = float(x.abs().max())
        for t, (slot, pos) in enumerate(rows):
            pg = int(table[slot, pos // page])
            assert float((q[t].cpu().double() - rotated(x[t, :H * D].reshape(H, D), pos)).abs().max()) < tol * scale
            got_k = k[pg, :, pos % page].cpu().double()
            assert float((got_k - rotated(x[t, H * D:(H + Kh) * D].reshape(Kh, D), pos)).abs().max()) < tol * scale
            got_v = v[pg, :, pos % page].cpu().double()
            assert float((got_v - x[t, (H + Kh) * D:].reshape(Kh, D)).abs().max()) < tol * scale

    check(ops32, 2e-6, 6, False)
    check(ops16, 6e-3, 6, False)
    check(ops16, 6e-3, 40, False)          # many tokens
    if 128 % D == 0:
        check(ops16, 6e-3, 5, True)


def test_scales_of_the_embedding_and_of_a_product(ops32, ops16):
    """The embedding's multiplier and a product's alpha: applied in the kernels, in float32."""
    g = torch.Generator(device="cuda").manual_seed(80)
    table = torch.randn(300, 272, device="cuda", generator=g)
    ids = torch.randint(0, 300, (9,), device="cuda", generator=g, dtype=torch.int32)
    assert torch.equal(ops32.embed(ids, table, 3.5), table[ids.long()] * 3.5)
    tb = table.to(BF16)
    assert torch.equal(ops16.embed(ids, tb, 0.25), tb[ids.long()].float() * 0.25)
    for ops, tol, shapes in ((ops32, 2e-6, [(5, 100, 33)]), (ops16, 6e-3, [(5, 200, 96), (8, 256, 4096), (300, 384, 520)])):
        for T, N, K in shapes:
            x = torch.randn(T, K, device="cuda", generator=g).to(ops.dtype)
            w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(ops.dtype)
            lw = ops.prepare_linear([w])
            ref = x.double() @ w.double().T
            assert _rel(ops.linear(x, lw, out_dtype=torch.float32, scale=0.3), ref * 0.3) < tol
            acc = torch.ones(T, N, device="cuda")
            ops.linear(x, lw, accumulate_into=acc, scale=-2.0)
            assert _rel(acc, 1.0 - 2.0 * ref) < tol
            plain_ = ops.linear(x, lw, out_dtype=torch.float32)
            assert torch.equal(ops.linear(x, lw, out_dtype=torch.float32, scale=1.0), plain_)


@pytest.mark.parametrize("T,N,K,share", [
    (300, 128, 8192, 4),        # one weight tile, its inner dimension in 32 parts
    (2048, 4096, 3584, 100),    # 32 weight tiles on 18 teams
    (2048, 4096, 14336, 0),     # the down product of a 2,048-token prompt, as the library plans it
    (2048, 520, 2056, 12),      # rows, and an inner size, that fill no tile
    (1000, 6144, 4096, 88), (257, 130, 1032, 4), (700, 1000, 4096, 12), (4100, 1032, 520, 12)])
def test_product_whose_weight_tiles_are_shared_between_teams(ops16, T, N, K, share):
    """More than 256 tokens, a product that is added to its output: the k blocks of all weight tiles
    are shared out among teams of CTAs (`share` blocks a team, asked for here; 0: what the library
    takes by itself), and a tile whose inner dimension two or more teams hold gets their parts added in
    the order of their k blocks.  Against float64 (with the stored and the gated product of the same
    sizes, which take tiles in turn); twice, bit for bit; the counters of finished parts back at zero;
    and the same without the counters (tiles in turn)."""
    import ctypes
    from ctypes import c_void_p
    from rbitnet_b200.kernels import ops as ops_module
    ops16.lib.call("rb_gemm_tc_share_for_test", share, launches=0)
    try:
        _shared_product_case(ops16, ops_module, T, N, K, share)
    finally:
        ops16.lib.call("rb_gemm_tc_share_for_test", 0, launches=0)


def _shared_product_case(ops16, ops_module, T, N, K, share):
    import ctypes
    from ctypes import c_void_p
    plan = (ctypes.c_int * 4)()
    sms = ops16.lib.raw("rb_device_sm_count")()
    ops16.lib.call("rb_gemm_tc_plan", T, N, K, 0, sms, 1, plan, launches=0)
    assert plan[1] > 0 and (share == 0 or plan[1] == share), "these sizes were chosen to share weight tiles"
    ws = ops_module._GEMM_WORKSPACES[torch.cuda.current_device()]
    counters = ws[:ops_module._GEMM_COUNTER_BYTES].view(torch.int32)
    g = torch.Generator(device="cuda").manual_seed(14)
    x = torch.randn(T, K, device="cuda", generator=g).to(BF16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(BF16)
    ref = x.double() @ w.double().T
    lw = ops16.prepare_linear([w])
    acc0 = torch.randn(T, N, device="cuda", generator=g)
    F = N // 2
    wg, wu = w[:F] * 2, w[F:2 * F]
    gate, up = x.double() @ wg.double().T, x.double() @ wu.double().T
    gu = ops16.prepare_gate_up(wg, wu)

    def run():
        stored = ops16.linear(x, lw, out_dtype=F32)
        acc = acc0.clone()
        ops16.linear(x, lw, accumulate_into=acc, scale=0.5)
        return stored, acc, ops16.gated_linear(x, gu)

    first = run()
    assert int(counters.abs().max()) == 0
    assert _rel(first[0], ref) < 2e-5
    assert _rel(first[1], acc0.double() + 0.5 * ref) < 2e-5
    assert _rel(first[2], gate / (1 + torch.exp(-gate)) * up) < 6e-3
    again = run()
    for a, b in zip(first, again):
        assert torch.equal(a, b)
    ops16.lib.call("rb_gemm_tc_set_workspace", c_void_p(0), 0, launches=0)
    try:
        in_turn = run()
    finally:
        ops16.lib.call("rb_gemm_tc_set_workspace", c_void_p(ws.data_ptr()), ws.numel(), launches=0)
    assert _rel(in_turn[0], ref) < 2e-5 and _rel(in_turn[1], acc0.double() + 0.5 * ref) < 2e-5
    assert _rel(in_turn[2], gate / (1 + torch.exp(-gate)) * up) < 6e-3
    assert int(counters.abs().max()) == 0
    ops16.check_errors()


@pytest.mark.parametrize("T,E,K,F", [(1, 256, 4096, 352), (5, 1000, 520, 176), (16, 4096, 1024, 1000),
                                     (33, 520, 2048, 352), (8, 4096, 14336, 2000)])
def test_norm_folded_into_the_products_around_it(ops16, T, E, K, F):
    """The product of up to 16 tokens that adds to the residual stream leaves the rows times the next
    norm's weights and their sums of squares; the stored, the added and the gated product take those and
    multiply their sums by each row's factor.  Each against float64, and against the norm kernel followed
    by the same product.  More tokens: nothing is left, and rows given with their norm pending are
    normed by the kernel of old."""
    from rbitnet_b200.kernels.ops import NormedRows
    g = torch.Generator(device="cuda").manual_seed(41)
    x0 = torch.randn(T, E, device="cuda", generator=g) * 2.0
    a = torch.randn(T, K, device="cuda", generator=g).to(BF16)
    w_o = (torch.randn(E, K, device="cuda", generator=g) / math.sqrt(K)).to(BF16)
    gw = 1.0 + 0.5 * torch.randn(E, device="cuda", generator=g)
    eps = 1e-5
    request = ops16.norm_request(gw, eps)
    assert request is not None
    x = x0.clone()
    ops16.linear(a, ops16.prepare_linear([w_o]), accumulate_into=x, then_norm=request)
    ref_x = x0.double() + a.double() @ w_o.double().T
    assert _rel(x, ref_x) < 2e-5
    rows = request.result
    assert (rows is not None) == (ops16._k_splits(T, E, K) >= 2 and T <= 16)
    plain = ops16.rmsnorm(x, gw, eps)                                      # the norm as a kernel of its own
    w1 = (torch.randn(F, E, device="cuda", generator=g) / math.sqrt(E)).to(BF16)
    lw1 = ops16.prepare_linear([w1])
    if rows is None:
        cut = torch.rand(5, T, device="cuda", generator=g)
        rows = NormedRows(x, gw, eps, (x * gw).to(BF16), ((cut / cut.sum(0)) * (x * x).sum(-1)).contiguous())
        assert torch.equal(ops16.linear(rows, lw1, out_dtype=F32), ops16.linear(plain, lw1, out_dtype=F32))
        return
    assert rows.x is x and rows.squares.shape[0] == 4 * -(-E // 128)
    assert _rel(rows.squares.sum(0), (x.double() ** 2).sum(-1)) < 1e-5
    assert _rel(rows.scaled, x.double() * gw.double()) < 4e-3             # one rounding to bfloat16
    factor = 1.0 / torch.sqrt((x.double() ** 2).mean(-1) + eps)
    h = rows.scaled.double() * factor[:, None]                             # what the next product should see
    assert _rel(plain, h) < 8e-3

    for N in (F, 4096):                     # few weight tiles (the inner dimension is split) and many
        w1 = (torch.randn(N, E, device="cuda", generator=g) / math.sqrt(E)).to(BF16)
        lw1 = ops16.prepare_linear([w1])
        ref = h @ w1.double().T
        assert _rel(ops16.linear(rows, lw1, out_dtype=F32), ref) < 2e-5
        assert _rel(ops16.linear(rows, lw1, out_dtype=F32, scale=0.25), 0.25 * ref) < 2e-5
        assert _rel(ops16.linear(plain, lw1, out_dtype=F32), ref) < 8e-3
        acc0 = torch.randn(T, N, device="cuda", generator=g)
        acc = acc0.clone()
        ops16.linear(rows, lw1, accumulate_into=acc)
        assert _rel(acc, acc0.double() + ref) < 2e-5
    wg = (torch.randn(F, E, device="cuda", generator=g) / math.sqrt(E) * 2).to(BF16)
    wu = (torch.randn(F, E, device="cuda", generator=g) / math.sqrt(E)).to(BF16)
    gate, up = h @ wg.double().T, h @ wu.double().T
    t = ops16.gated_linear(rows, ops16.prepare_gate_up(wg, wu))
    assert _rel(t, gate / (1 + torch.exp(-gate)) * up) < 6e-3
    ops16.check_errors()


@pytest.mark.parametrize("T,F,K", [(512, 14336, 2048), (300, 14336, 2048), (300, 14330, 4096)])
def test_a_last_round_of_few_tiles_becomes_a_product_of_its_own(ops16, T, F, K):
    """Tiles that are a few more than whole rounds of the SMs (448 = 3 x 148 + 4 here): the weight tiles of
    the whole rounds stay one product, the few that are left become a second one with token tiles of 64
    whose K is cut into a cluster; the gated product (whose cluster sum pairs gate and up) and the stored
    one, against float64, with and without the second product."""
    sms = ops16.lib.raw("rb_device_sm_count")()
    if sms != 148:
        pytest.skip("the sizes are chosen for 148 SMs")
    g = torch.Generator(device="cuda").manual_seed(15)
    x = torch.randn(T, K, device="cuda", generator=g).to(BF16)
    wg = (torch.randn(F, K, device="cuda", generator=g) / math.sqrt(K) * 2).to(BF16)
    wu = (torch.randn(F, K, device="cuda", generator=g) / math.sqrt(K)).to(BF16)
    gate, up = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = gate / (1 + torch.exp(-gate)) * up
    gu = ops16.prepare_gate_up(wg, wu)
    ws = torch.cat([wg, wu])[:28672]
    lw = ops16.prepare_linear([ws])
    want_s = x.double() @ ws.double().T
    launched = ops16.lib.raw("rb_gemm_tc_kernels_launched")
    got, kernels = {}, {}
    try:
        for mode in (0, -1):
            ops16.lib.call("rb_gemm_tc_tail_for_test", mode, launches=0)
            before = launched()
            got[mode] = (ops16.gated_linear(x, gu), ops16.linear(x, lw, out_dtype=F32))
            kernels[mode] = launched() - before
    finally:
        ops16.lib.call("rb_gemm_tc_tail_for_test", 0, launches=0)
    # both products in two kernels each; but a gated output whose rows TMA cannot address (14,330 bfloat16
    # values) takes token tiles of 64 from the start, in one kernel
    assert kernels[-1] == 2 and kernels[0] == (4 if F % 8 == 0 else 3), kernels
    for mode in (0, -1):
        assert _rel(got[mode][0], want) < 6e-3
        assert _rel(got[mode][1], want_s) < 2e-5
    ops16.check_errors()
