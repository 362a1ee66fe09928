"""Host-side choices the kernel library makes, asked without a GPU: into how many parts the keys of a
decode are cut and when those parts merge on chip, which sizes each kernel says it takes, and which
requests are refused with a message.  The library is built by nvcc where it is missing (no device is
needed to build or to load it); without nvcc these tests are skipped."""
import shutil

import pytest

if shutil.which("nvcc") is None:
    pytest.skip("nvcc is not installed here", allow_module_level=True)


@pytest.fixture(scope="module")
def lib():
    from rbitnet_b200.kernels.lib import load
    return load(verbose=False)


@pytest.mark.parametrize("D", [64, 128])
def test_parts_of_a_decode(lib, D):
    parts, on_chip = lib.raw("rb_attention_decode_tma_parts"), lib.raw("rb_attention_decode_tma_on_chip")
    for pairs in (1, 7, 8, 32, 64, 100, 256, 300, 512, 600, 1024, 5000):
        for tiles in (1, 2, 3, 5, 16, 33, 128):
            s = parts(pairs, tiles, D)
            assert 1 <= s <= min(16, tiles), (pairs, tiles, s)          # no part without a tile to start from
            if on_chip(pairs, s, D):
                assert s in (2, 4, 8, 16)                               # cluster sizes
        assert parts(pairs, 1, D) == 1
    # a small batch is cut as far as its context allows, and merges on chip (up to 8 parts on any device)
    assert parts(8, 4, D) == 4 and on_chip(8, 4, D)
    assert parts(64, 32, 128) == 4 and on_chip(64, 4, 128)
    assert parts(0, 5, D) == 1 and parts(5, 0, D) == 1
    # more CTAs fit an SM at head size 64, so more pairs still count as a small grid
    assert parts(256, 32, 64) == 2 and parts(256, 32, 128) == 1
    assert not on_chip(600, 4, D)


def test_sizes_the_kernels_take(lib):
    assert lib.raw("rb_attention_decode_tma_supports")(32, 8, 128, 64)
    assert not lib.raw("rb_attention_decode_tma_supports")(32, 8, 96, 64)      # head size
    assert not lib.raw("rb_attention_decode_tma_supports")(32, 8, 128, 16)     # pages of 16 positions
    assert not lib.raw("rb_attention_decode_tma_supports")(34, 2, 128, 64)     # 17 query heads a group
    assert lib.raw("rb_attention_prefill_tc_supports")(32, 8, 64, 128)
    assert not lib.raw("rb_attention_prefill_tc_supports")(7, 2, 128, 64)      # heads that are no multiple of the groups
    assert lib.raw("rb_attention_tiled_supports")(6, 2, 96, 64, 1)
    assert not lib.raw("rb_attention_tiled_supports")(6, 2, 100, 64, 1)
    assert lib.raw("rb_gemm_tc_qkv_supports")(8, 128, 4)
    assert not lib.raw("rb_gemm_tc_qkv_supports")(8, 128, 1)                   # K has to be split
    assert not lib.raw("rb_gemm_tc_qkv_supports")(17, 128, 4)                  # few tokens only
    assert not lib.raw("rb_gemm_tc_qkv_supports")(8, 96, 4)                    # a head may not straddle two tiles


def test_requests_are_refused_with_a_message(lib):
    from rbitnet_b200.kernels.lib import KernelError
    with pytest.raises(KernelError, match="multiple of 8"):
        lib.call("rb_gemm_tc", 0, 50, 1, 0, 77, 9, 0, 77, 50, 50, 77, 0, 0, 1, 0, 1.0, 0)
    with pytest.raises(KernelError, match="rows in blocks of 32"):
        lib.call("rb_gemm_tc", 0, 64, 1, 0, 64, 8, 0, 64, 48, 48, 128, 3, 24, 1, 0, 1.0, 0)
    with pytest.raises(KernelError, match="at most 8 splits"):
        lib.call("rb_gemm_tc", 0, 64, 1, 0, 1024, 8, 0, 1024, 64, 64, 1024, 0, 0, 9, 0, 1.0, 0)
    with pytest.raises(KernelError, match="head_dim"):
        lib.call("rb_rotate_append", 0, 0, 0, 1, 0, 0, 0, 0, 0, 0, 1, 64, 1, 2, 1, 7, 1, 7, 0, 0)


def test_parts_of_a_product_and_of_the_plain_decode(lib):
    """The choices follow the device's SM count (148 where no device answers, as here without a GPU)."""
    splits, parts = lib.raw("rb_gemm_tc_splits"), lib.raw("rb_attention_decode_parts")
    sms = lib.raw("rb_device_sm_count")()
    assert sms > 0
    assert splits(300, 4096, 4096) == 1                      # beyond 256 tokens K stays whole
    for T, N, K in [(1, 4096, 4096), (8, 6144, 4096), (8, 4096, 14336), (64, 128256, 4096), (16, 64, 64),
                    (200, 4096, 4096), (8, 256, 320)]:
        s = splits(T, N, K)
        blocks = -(-K // 64)
        assert s in range(1, 9) and (s - 1) * -(-blocks // s) < blocks, (T, N, K, s)     # no part is empty
        tiles = -(-N // 128) * -(-T // 64)
        assert s == 1 or tiles * 2 <= 2 * sms                # K is cut only while CTAs are fewer than places
    if sms == 148:
        assert splits(8, 4096, 4096) == 8 and splits(8, 6144, 4096) == 4 and splits(8, 128256, 4096) == 1
    for batch, kvh, ctx in [(1, 8, 2048), (8, 8, 2048), (64, 8, 8192), (3, 1, 10), (500, 8, 4096)]:
        s = parts(batch, kvh, ctx)
        assert 1 <= s <= min(16, max(1, -(-ctx // 64))), (batch, kvh, ctx, s)
    assert parts(1, 1, 64) == 1 and parts(0, 8, 100) == 1


def _plan(lib, T, N, K, sms=148, workspace=1, tile=0):
    import ctypes
    out = (ctypes.c_int * 4)()
    lib.call("rb_gemm_tc_plan", T, N, K, tile, sms, workspace, out, launches=0)
    return dict(tile=out[0], blocks_per_team=out[1], teams=out[2], token_tiles=out[3])


def test_plan_of_a_product_of_many_tokens(lib):
    """Tiles in turn, or (a product added to its output, on a device that has the counters: `workspace`)
    the k blocks of all weight tiles shared out evenly among teams of CTAs."""
    # 2,048 tokens, 4,096 rows: 256 tiles are 1.73 rounds of 148 SMs; 18 teams of 8 CTAs share 32 weight tiles
    p = _plan(lib, 2048, 4096, 14336)
    assert p["tile"] == 256 and p["token_tiles"] == 8 and p["teams"] == 18
    assert p["blocks_per_team"] * 18 >= 32 * 224 > p["blocks_per_team"] * 17 and p["blocks_per_team"] % 4 == 0
    # without the counters, and for few tokens, tiles are taken in turn
    assert _plan(lib, 2048, 4096, 14336, workspace=0)["blocks_per_team"] == 0
    assert _plan(lib, 64, 4096, 4096)["blocks_per_team"] == 0 and _plan(lib, 64, 4096, 4096)["tile"] == 64
    # tiles that fill whole rounds stay as they are: 37 weight tiles x 8 token tiles = 2 x 148
    assert _plan(lib, 2048, 37 * 128, 4096)["blocks_per_team"] == 0
    # few tiles and a long inner dimension: every SM gets a share of some tile's inner dimension
    p = _plan(lib, 300, 4096, 14336)
    assert p["tile"] == 160 and p["token_tiles"] == 2 and p["teams"] > 64 and p["blocks_per_team"] > 0
    # the parts of a tile are added one after the other: not worth it where the products are short
    assert _plan(lib, 2048, 4096, 4096)["blocks_per_team"] == 0
    # every part is at least one block, and the teams cover everything, at any size
    for T in (129, 257, 300, 1000, 2048, 4097, 9000):
        for N in (128, 130, 4096, 6144, 28672, 128256):
            for K in (64, 72, 4096, 14336):
                for sms in (148, 132, 16):
                    p = _plan(lib, T, N, K, sms=sms)
                    w_tiles, blocks = -(-N // 128), -(-K // 64)
                    assert p["tile"] in (128, 160, 192, 224, 256) and p["token_tiles"] == -(-T // p["tile"])
                    if p["blocks_per_team"]:
                        assert p["teams"] * p["token_tiles"] <= sms
                        assert p["teams"] * p["blocks_per_team"] >= w_tiles * blocks > (p["teams"] - 1) * p["blocks_per_team"]
