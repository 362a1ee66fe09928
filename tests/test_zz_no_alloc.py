"""The decode-attention entry point that allocates nothing (rb_attention_decode_static).

Some programs that embed this library cannot allocate device memory at the time they call it:
they run inside a memory budget fixed at start-up, or inside a host that owns the allocator, or
in a loop where an allocation is not allowed.  For them the split decode's scratch lives in a
static device array inside the library.  This test calls that entry point through its exported
C symbol and checks it against the ordinary entry point (caller-provided scratch) on two calls
in a row with different inputs, so that what the first call left in the shared array cannot
help or hurt the second.  The file sorts last on purpose: a run that stops at the first
failure has by then run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(t.data_ptr())


def test_static_scratch_decode_matches_the_allocating_entry_point():
    from rbitnet_b200.kernels.lib import load
    lib = load()
    dll = ctypes.CDLL(lib.path)                       # the exported C symbols, nothing else
    static = dll.rb_attention_decode_static
    static.restype = c_int
    static.argtypes = [c_void_p] * 5 + [c_int, c_int, c_void_p, c_void_p] + [c_int] * 4 + [c_float, c_int, c_int, c_void_p]
    plain = dll.rb_attention_decode
    plain.restype = c_int
    plain.argtypes = [c_void_p] * 5 + [c_int, c_int, c_void_p, c_void_p] + [c_int] * 4 + [c_float, c_int,
                                                                                       c_void_p, c_void_p, c_int, c_void_p]
    dll.rb_last_error.restype = ctypes.c_char_p
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    H, Kh, D, page, n_slots, max_pages = 8, 2, 64, 64, 4, 8
    for call, (lens, splits, window) in enumerate([([500, 64, 1, 130], 5, 0), ([33, 512, 257, 90], 3, 100)]):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        k = torch.randn(n_slots * max_pages, Kh, page, D, device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn(n_slots * max_pages, Kh, page, D, device="cuda", generator=g).to(torch.bfloat16)
        table = torch.randperm(n_slots * max_pages).to(torch.int32).reshape(n_slots, max_pages).cuda()
        B = len(lens)
        q = (torch.randn(B, H, D, device="cuda", generator=g) * 2).to(torch.bfloat16)
        pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
        slot = torch.arange(B, dtype=torch.int32, device="cuda")
        scale = 1.0 / math.sqrt(D)
        want = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
        part_o = torch.empty(B, H, splits, D, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(B, H, splits, 2, dtype=torch.float32, device="cuda")
        rc = plain(_ptr(want), _ptr(q), _ptr(k), _ptr(v), _ptr(table), max_pages, page, _ptr(pos), _ptr(slot),
                   B, H, Kh, D, scale, window, _ptr(part_o), _ptr(part_ml), splits, stream)
        assert rc == 0, dll.rb_last_error()
        got = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()     # what the driver has left: any allocation would show here
        rc = static(_ptr(got), _ptr(q), _ptr(k), _ptr(v), _ptr(table), max_pages, page, _ptr(pos), _ptr(slot),
                    B, H, Kh, D, scale, window, splits, stream)
        assert rc == 0, dll.rb_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call > 0:        # the first call on the device loads the kernels and looks the array up; later ones take nothing
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert torch.isfinite(got.float()).all()
        err = float((got.double() - want.double()).abs().max()) / float(want.double().abs().max())
        assert err < 8e-3, (call, err)                 # the tolerance of the attention kernel tests
        # and against the definition, so that both being wrong together would show
        for b, n in enumerate(lens):
            lo = max(0, n - window) if window else 0
            idx = torch.arange(lo, n, device="cuda")
            pages = table[b, (idx // page).long()].long()
            for h in (0, H - 1):
                kk = k[pages, h // (H // Kh), (idx % page).long()].double()
                vv = v[pages, h // (H // Kh), (idx % page).long()].double()
                ref = torch.softmax((kk @ q[b, h].double()) * scale, 0) @ vv
                e = float((got[b, h * D:(h + 1) * D].double() - ref).abs().max()) / float(ref.abs().max())
                assert e < 8e-3, (call, b, h, e)

    # one part needs no scratch: the same call with n_splits = 1 is served whatever the limit says
    rc = static(_ptr(got), _ptr(q), _ptr(k), _ptr(v), _ptr(table), max_pages, page, _ptr(pos), _ptr(slot),
                B, H, Kh, D, scale, window, 1, stream)
    assert rc == 0, dll.rb_last_error()
    torch.cuda.synchronize()
    assert float((got.double() - want.double()).abs().max()) / float(want.double().abs().max()) < 8e-3

    # a size beyond the static array is refused with a clear message, and nothing is launched
    rc = static(_ptr(got), _ptr(q), _ptr(k), _ptr(v), _ptr(table), max_pages, page, _ptr(pos), _ptr(slot),
                4096, 64, Kh, 128, scale, 0, 32, stream)
    assert rc != 0 and b"exceed the static" in dll.rb_last_error()
