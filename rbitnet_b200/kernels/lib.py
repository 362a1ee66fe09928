"""Loads the built kernel library and declares its C entry points.

There is no other implementation behind these calls: if the library cannot be
built or loaded, ``load()`` raises, and so does everything that needs a kernel.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_float, c_void_p, c_char_p
from typing import Optional

from .build import library_path

P, I, L, F = c_void_p, c_int, c_int64, c_float

_SIGNATURES = {
    "rb_abi_version": [],
    "rb_embed": [P, P, I, P, I, I, I, F, P],
    "rb_rmsnorm": [P, I, P, P, I, I, F, P],
    "rb_rotate_append": [P, P, L, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P],
    "rb_silu_mul": [P, P, I, I, I, I, L, I, P],
    "rb_gather_rows": [P, P, P, I, I, P],
    "rb_gemm_simple": [P, L, I, P, L, P, L, I, I, I, I, I, F, P],
    "rb_attention_simple": [P, P, I, P, P, P, I, I, P, P, I, I, I, I, F, I, P],
    "rb_sample": [P, P, L, I, I, P, P, P, P],
    "rb_sample_chunks": [I],
    "rb_gemm_tc": [P, L, I, P, L, I, P, L, I, I, I, I, I, I, I, F, P],
    "rb_gemm_tc_qkv": [P, P, L, I, P, L, I, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P],
    "rb_read_error_flag": [P, I],
    "rb_decode_advance": [P, P, P, I, P, P, P, P, P],
    "rb_error_flag_addresses": [P, P],
    "rb_attention_prefill": [P, P, P, P, P, I, I, P, P, P, P, I, I, I, I, F, I, P],
    "rb_attention_decode": [P, P, P, P, P, I, I, P, P, I, I, I, I, F, I, P, P, I, P],
    "rb_attention_prefill_tc": [P, P, P, P, L, P, I, I, P, P, P, P, I, I, I, I, F, I, P],
    "rb_attention_decode_tma": [P, P, P, P, L, P, I, I, P, P, I, I, I, I, F, I, P, P, I, P],
    "rb_attention_decode_static": [P, P, P, P, P, I, I, P, P, I, I, I, I, F, I, I, P],
    "rb_set_error_flag_for_test": [I],
    "rb_wait_probe": [L, I, P, P],
    "rb_count_wait_probe": [P, L, I, P, P],
}


#: source files whose kernels address the cache through the checked function (each has its own word)
CHECKED_FILES = ("elementwise", "gemm_tcgen05", "attention_simple", "attention_tiled")


class KernelError(RuntimeError):
    pass


class KernelLibrary:
    def __init__(self, path):
        self.path = str(path)
        self._dll = ctypes.CDLL(self.path)
        self._dll.rb_last_error.restype = c_char_p
        self._dll.rb_last_error.argtypes = []
        self.launches = 0   # kernels launched through this library, for the bench's record
        for name, argtypes in _SIGNATURES.items():
            self.declare(name, argtypes)
        self.declare("rb_attention_tiled_supports", [I, I, I, I, I])
        self.declare("rb_attention_prefill_tc_supports", [I, I, I, I])
        self.declare("rb_gemm_tc_qkv_supports", [I, I, I])
        self.declare("rb_attention_decode_tma_supports", [I, I, I, I])
        self.declare("rb_attention_decode_tma_parts", [I, I, I])
        self.declare("rb_attention_decode_tma_on_chip", [I, I, I])
        self.declare("rb_attention_decode_parts", [I, I, I])
        self.declare("rb_gemm_tc_splits", [I, I, I])
        self.declare("rb_gemm_tc_workspace_bytes", [], restype=ctypes.c_longlong)
        self.declare("rb_gemm_tc_set_workspace", [P, L])
        self.declare("rb_gemm_tc_plan", [I, I, I, I, I, I, P])
        self.declare("rb_gemm_tc_share_for_test", [I])
        self.declare("rb_gemm_tc_tail_for_test", [I])
        self.declare("rb_gemm_tc_kernels_launched", [])
        self.declare("rb_gemm_tc_pending_norm", [P, I, F, F])
        self.declare("rb_gemm_tc_leave_norm", [P, L, P, P])
        self.declare("rb_gemm_tc_norm_parts", [I])
        self.declare("rb_device_sm_count", [])
        self.declare("rb_is_checked_build", [])
        for tu in CHECKED_FILES:
            self.declare(f"rb_check_word_{tu}", [P, I])

    def declare(self, name, argtypes, restype=c_int):
        fn = getattr(self._dll, name)
        fn.argtypes = argtypes
        fn.restype = restype
        return fn

    def has(self, name) -> bool:
        return hasattr(self._dll, name)

    def call(self, name, *args, launches: int = 1):
        rc = getattr(self._dll, name)(*args)
        if rc != 0:
            raise KernelError(self._dll.rb_last_error().decode(errors="replace") or f"{name} failed ({rc})")
        self.launches += launches

    def raw(self, name):
        return getattr(self._dll, name)


_LIB: Optional[KernelLibrary] = None


def load(verbose: bool = True) -> KernelLibrary:
    """The library for the current build flags (RBITNET_CHECKED selects the checked build)."""
    global _LIB
    path = library_path(verbose=verbose)
    if _LIB is None or _LIB.path != str(path):
        _LIB = KernelLibrary(path)
    return _LIB
