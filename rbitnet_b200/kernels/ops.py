"""The operations a step is made of, on device tensors, each one a launch of this
package's own CUDA kernels.

``CudaOps(dtype)`` is the only implementation on the product path.  With
``torch.float32`` every product is a float32 FFMA sum and every activation,
cache entry and weight is float32 (no tensor-core or reduced-precision mode).
With ``torch.bfloat16`` weights, activations between kernels and the cache are
bfloat16, while the residual stream, norms, rotation angles, softmax and all
accumulation stay float32.
"""
from __future__ import annotations

from ctypes import c_void_p
from dataclasses import dataclass
from typing import List, Optional

import torch

from .lib import load, KernelError

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


@dataclass
class LinearWeight:
    """A weight matrix [out, in] made ready for ``linear``."""
    w: torch.Tensor
    n_out: int
    n_in: int


@dataclass
class GateUpWeight:
    """Gate and up matrices made ready for ``gated_linear``.

    ``block == 0``: rows [gate | up].  ``block == 16``: for every 16 output features, their 16 gate
    rows followed by their 16 up rows (the last group padded with zero rows), which is how the
    tensor-core product pairs gate and up inside one warp of its epilogue."""
    w: torch.Tensor
    inner: int
    n_in: int
    block: int = 0


@dataclass
class NormRequest:
    """Asks the product that adds to the residual stream to leave what the norm after it needs
    (``CudaOps.linear(..., then_norm=request)``).  ``result`` is the ``NormedRows`` if it did."""
    weight: torch.Tensor          # float32 [width]
    eps: float
    result: Optional["NormedRows"] = None


@dataclass
class NormedRows:
    """Rows of the residual stream with an RMS norm pending: a product that takes them multiplies its
    finished sums by each row's 1/sqrt(mean of squares + eps) (``CudaOps.linear``, ``gated_linear`` and
    ``project_rotate_append`` take them in place of the normed rows; ``CudaOps.normed`` gives the normed
    rows themselves).  The norm is the same float32 arithmetic either way; what is rounded to bfloat16
    is row * weight instead of row * factor * weight."""
    x: torch.Tensor               # the rows themselves, float32 [T, width]
    weight: torch.Tensor          # float32 [width]
    eps: float
    scaled: torch.Tensor          # bfloat16 [T, width]: x * weight
    squares: torch.Tensor         # float32 [parts, T]: sums of squares of x over parts of the width

    @property
    def shape(self):
        return self.x.shape


#: per device: the workspace of the tensor-core products (arrival counters, then partial sums of
#: tiles whose inner dimension is shared between teams of CTAs).  One per process and device, never
#: freed: the library keeps its address.
_GEMM_WORKSPACES = {}
_GEMM_WORKSPACE_SET = set()
_GEMM_COUNTER_BYTES = 4 << 16


def _give_gemm_workspace(lib, device: torch.device) -> None:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if (lib.path, index) in _GEMM_WORKSPACE_SET:
        return
    with torch.cuda.device(index):
        ws = _GEMM_WORKSPACES.get(index)
        if ws is None:
            n = int(lib.raw("rb_gemm_tc_workspace_bytes")())
            ws = _GEMM_WORKSPACES[index] = torch.zeros(n, dtype=torch.uint8, device=device)
            torch.cuda.synchronize(index)
        lib.call("rb_gemm_tc_set_workspace", c_void_p(ws.data_ptr()), ws.numel(), launches=0)
    _GEMM_WORKSPACE_SET.add((lib.path, index))


class CudaOps:
    def __init__(self, dtype=torch.bfloat16, device="cuda:0", verbose_build: bool = True):
        if dtype not in _CODE:
            raise ValueError(f"compute dtype must be float32 or bfloat16, found {dtype}")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: rbitnet_b200 runs its kernels on a B200 and has no other path")
        self.dtype = dtype
        self.code = _CODE[dtype]
        self.device = torch.device(device)
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"device {self.device} has compute capability {major}.{minor}; "
                              "the kernels are built for sm_100a only")
        self.lib = load(verbose=verbose_build)
        #: prefill attention of head sizes 64 and 128 runs on tcgen05 (else on the mma.sync kernel)
        self.prefill_on_tcgen05 = True
        #: decode attention of head sizes 64 and 128 gets its keys and values by TMA (else by cp.async)
        self.decode_on_tma = True
        self._flag_ptrs = None
        #: a decode step's norms between two products are folded into them (see ``NormedRows``)
        self.fold_norms = True
        self.fold_norms_up_to = 16
        #: tensor-core products of more than 256 tokens may share a weight tile's inner dimension
        #: between teams of CTAs (needs the workspace; tiles are taken in turn without it)
        _give_gemm_workspace(self.lib, self.device)

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, t: torch.Tensor, dtype, what: str):
        if t.dtype != dtype or not t.is_cuda or not t.is_contiguous():
            raise KernelError(f"{what}: expected a contiguous {dtype} CUDA tensor, found {t.dtype} "
                              f"on {t.device}, contiguous={t.is_contiguous()}")

    def check_errors(self) -> None:
        """Raises if a kernel recorded that one of its bounded waits ran out."""
        import ctypes
        v = ctypes.c_int(0)
        self.lib.call("rb_read_error_flag", ctypes.byref(v), 1, launches=0)
        if v.value:
            ws = _GEMM_WORKSPACES.get(self.device.index if self.device.index is not None else torch.cuda.current_device())
            if ws is not None:
                ws[:_GEMM_COUNTER_BYTES].zero_()      # a product that gave up may have left counts behind
            raise KernelError(f"a kernel gave up waiting (code {v.value}: 1 = loader, 2 = tensor-core issuer, "
                              "3 = epilogue, 4 = the parts of a shared weight tile); its results are not valid")
        if self.lib.raw("rb_is_checked_build")():
            from .lib import CHECKED_FILES
            w = (ctypes.c_int * 4)()
            for tu in CHECKED_FILES:
                self.lib.call(f"rb_check_word_{tu}", w, 1, launches=0)
                if w[0]:
                    raise KernelError(f"checked build ({tu}): a kernel asked for slot {w[1]}, position {w[2]}, kv head "
                                      f"{w[3]}, which lies outside the cache (code {w[0]}); the access was not made")

    def to_compute(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    # ------------------------------------------------------------------ weights
    def prepare_embedding(self, table: torch.Tensor) -> torch.Tensor:
        return self.to_compute(table)

    def prepare_linear(self, weights: List[torch.Tensor]) -> LinearWeight:
        """One matrix from the given ones stacked along the output axis."""
        if len(weights) == 1:
            w = self.to_compute(weights[0])
        else:
            w = torch.cat([self.to_compute(x) for x in weights], dim=0).contiguous()
        return LinearWeight(w, w.shape[0], w.shape[1])

    def rows_of(self, weight: LinearWeight, first: int, count: int) -> LinearWeight:
        """Output rows first .. first+count-1 of a prepared matrix, sharing its memory."""
        return LinearWeight(weight.w[first:first + count], count, weight.n_in)

    def prepare_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> GateUpWeight:
        gate, up = self.to_compute(gate), self.to_compute(up)
        F, K = gate.shape
        if self.dtype == torch.bfloat16 and K % 8 == 0:
            # the layout of the tensor-core gated product: groups of 16 gate rows and their 16 up rows
            groups = -(-F // 16)
            w = torch.zeros((groups, 2, 16, K), dtype=gate.dtype, device=gate.device)
            for half, m in ((0, gate), (1, up)):
                whole = F // 16
                w[:whole, half] = m[:whole * 16].view(whole, 16, K)
                if F % 16:
                    w[whole, half, :F % 16] = m[whole * 16:]
            return GateUpWeight(w.view(groups * 32, K), F, K, 16)
        return GateUpWeight(torch.cat([gate, up], dim=0).contiguous(), F, K, 0)

    # ------------------------------------------------------------------ ops
    def embed(self, ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """float32 rows table[ids] * scale."""
        T, (V, E) = ids.shape[0], table.shape
        out = torch.empty((T, E), dtype=torch.float32, device=self.device)
        self.lib.call("rb_embed", _ptr(out), _ptr(table), _CODE[table.dtype], _ptr(ids), T, E, V, float(scale),
                      self._stream())
        return out

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype=None) -> torch.Tensor:
        self._check(x, torch.float32, "rmsnorm input")
        T, E = x.shape
        out = torch.empty((T, E), dtype=out_dtype or self.dtype, device=self.device)
        self.lib.call("rb_rmsnorm", _ptr(out), _CODE[out.dtype], _ptr(x), _ptr(w), T, E, float(eps), self._stream())
        return out

    def linear(self, x, weight: LinearWeight, out_dtype=None, accumulate_into: Optional[torch.Tensor] = None,
               scale: float = 1.0, then_norm: Optional[NormRequest] = None) -> torch.Tensor:
        """scale * x[T, in] * W[out, in]^T (the scale multiplies the finished float32 sums).  With
        ``accumulate_into`` (float32 [T, out]) the product is added to it in float32 and it is returned.
        ``x`` may be ``NormedRows``.  ``then_norm``: see ``NormRequest`` (granted for a few tokens, where
        the product's parts along the inner dimension meet on chip)."""
        pending = x if isinstance(x, NormedRows) else None
        if pending is not None:
            if self._takes_pending(pending, weight.w):
                x = pending.scaled
            else:
                x, pending = self.normed(pending), None
        self._check(x, self.dtype, "linear input")
        T, K = x.shape
        if K != weight.n_in:
            raise KernelError(f"linear: input width {K} does not match the weight's {weight.n_in}")
        N = weight.n_out
        if accumulate_into is not None:
            out, acc = accumulate_into, 1
            self._check(out, torch.float32, "linear accumulate_into")
        else:
            out, acc = torch.empty((T, N), dtype=out_dtype or self.dtype, device=self.device), 0
        if self._tensor_core_ok(x, weight.w):
            # few tokens and few weight tiles: K is cut into parts so that every SM streams a piece
            # of W; the parts of a tile are one thread-block cluster and are summed on chip
            splits = self._k_splits(T, N, K)
            if pending is not None:
                self._pending_norm(pending)
            # (up to 16 tokens: measured at batch 1 and 8 a step gains 2.8 and 1.5 %, at batch 64 it loses 1 %:
            # the norm's kernel also was the time in which the next product's first tiles of W arrived)
            if then_norm is not None and acc and splits >= 2 and T <= self.fold_norms_up_to and out.is_contiguous():
                then_norm.result = self._leave_norm(out, then_norm, T, N)
            self.lib.call("rb_gemm_tc", _ptr(out), out.stride(0), _CODE[out.dtype], _ptr(x), x.stride(0), T,
                          _ptr(weight.w), weight.w.stride(0), N, N, K, acc, 0, splits,
                          64 if 64 < T <= 256 else 0, float(scale), self._stream())
        else:
            self.lib.call("rb_gemm_simple", _ptr(out), out.stride(0), _CODE[out.dtype], _ptr(x), x.stride(0),
                          _ptr(weight.w), weight.w.stride(0), self.code, T, N, K, acc, float(scale), self._stream())
        return out

    # ------------------------------------------------------------------ a norm between two products
    def norm_request(self, weight: torch.Tensor, eps: float) -> Optional[NormRequest]:
        """A request for ``linear(..., then_norm=)``, or None where norms are not folded into products
        (the float32 path keeps every norm a kernel of its own)."""
        if self.dtype != torch.bfloat16 or not self.fold_norms:
            return None
        return NormRequest(weight, float(eps))

    def normed(self, rows: NormedRows) -> torch.Tensor:
        """The normed rows themselves, for whoever does not take ``NormedRows``."""
        return self.rmsnorm(rows.x, rows.weight, rows.eps)

    def _takes_pending(self, rows: NormedRows, w: torch.Tensor) -> bool:
        return (self.dtype == torch.bfloat16 and rows.scaled.shape[0] <= 16 and self._tensor_core_ok(rows.scaled, w))

    def _pending_norm(self, rows: NormedRows) -> None:
        """For the next tensor-core product of this thread."""
        self.lib.call("rb_gemm_tc_pending_norm", _ptr(rows.squares), rows.squares.shape[0], float(rows.x.shape[1]),
                      float(rows.eps), launches=0)

    def _leave_norm(self, out: torch.Tensor, request: NormRequest, T: int, N: int) -> NormedRows:
        """For the next tensor-core product of this thread (one that adds into ``out``)."""
        parts = self.lib.raw("rb_gemm_tc_norm_parts")(N)
        scaled = torch.empty((T, N), dtype=torch.bfloat16, device=self.device)
        squares = torch.empty((parts, T), dtype=torch.float32, device=self.device)
        self.lib.call("rb_gemm_tc_leave_norm", _ptr(scaled), scaled.stride(0), _ptr(request.weight), _ptr(squares),
                      launches=0)
        return NormedRows(out, request.weight, request.eps, scaled, squares)

    def _k_splits(self, T: int, N: int, K: int) -> int:
        """Parts to cut the inner dimension into: the library's choice for this device (1 beyond 256
        tokens; else up to 8, so that every SM streams a piece of W)."""
        return self.lib.raw("rb_gemm_tc_splits")(T, N, K)

    def _tensor_core_ok(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        """The tcgen05 product takes bfloat16 operands whose rows TMA can address: inner size and
        row strides multiples of 8 elements, 16-byte aligned bases.  Anything else runs on the
        plain product."""
        return (self.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
                and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and x.stride(1) == 1 and w.stride(1) == 1)

    def gated_linear(self, x: torch.Tensor, weight: GateUpWeight) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) -> [T, inner] in the compute dtype."""
        pending = x if isinstance(x, NormedRows) else None
        if pending is not None:
            if weight.block == 16 and self._takes_pending(pending, weight.w):
                x = pending.scaled
            else:
                x, pending = self.normed(pending), None
        T = x.shape[0]
        out = torch.empty((T, weight.inner), dtype=self.dtype, device=self.device)
        rows = weight.w.shape[0]
        if weight.block == 16 and self._tensor_core_ok(x, weight.w):
            # one accumulator per tile; gate and up of a feature meet in the epilogue, and the
            # activation and the product happen on the way out
            if pending is not None:
                self._pending_norm(pending)
            self.lib.call("rb_gemm_tc", _ptr(out), out.stride(0), self.code, _ptr(x), x.stride(0), T,
                          _ptr(weight.w), weight.w.stride(0), rows, rows, weight.n_in, 3, weight.inner, 1, 0,
                          1.0, self._stream())
            return out
        gu = self.linear(x, LinearWeight(weight.w, rows, weight.n_in))
        self.lib.call("rb_silu_mul", _ptr(out), _ptr(gu), self.code, self.code, T, weight.inner, gu.stride(0),
                      weight.block, self._stream())
        return out

    def rotate_append(self, qkv: torch.Tensor, rotary, meta, view, n_heads: int) -> torch.Tensor:
        """Rotates q (and k) by position, appends k and v to the cache; returns q [T, H, D]."""
        D, Kh = view.head_dim, view.n_kv_heads
        T, width = qkv.shape
        if rotary is None:
            inv_freq, interleaved, rot_dim = self._zeros_freq(D), False, D
        else:
            inv_freq, interleaved, rot_dim = rotary
        want = (n_heads + (2 * Kh if view.writes else 0)) * D
        if width != want:
            raise KernelError(f"rotate_append: rows of {width} values, expected {want}")
        q = torch.empty((T, n_heads, D), dtype=self.dtype, device=self.device)
        self.lib.call("rb_rotate_append", _ptr(q), _ptr(qkv), qkv.stride(0), self.code, _ptr(inv_freq),
                      _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(view.k), _ptr(view.v), _ptr(view.page_table),
                      view.max_pages, view.page_size, T, n_heads, Kh, D, 1 if view.writes else 0, rot_dim,
                      1 if interleaved else 0, self._stream())
        return q

    def project_rotate_append(self, h: torch.Tensor, weight: LinearWeight, rotary, meta, view,
                              n_heads: int) -> torch.Tensor:
        """q/k/v product of the normed rows ``h``, rotation by position and cache append; returns the
        rotated q [T, H, D].  For a few tokens (a decode step) the product's own epilogue rotates and
        appends, from its float32 sums; otherwise the product is stored and ``rotate_append`` follows."""
        pending = h if isinstance(h, NormedRows) else None
        if pending is not None:
            if self._takes_pending(pending, weight.w):
                h = pending.scaled
            else:
                h, pending = self.normed(pending), None
        T, K = h.shape
        D, Kh = view.head_dim, view.n_kv_heads
        splits = self._k_splits(T, weight.n_out, K)
        if rotary is None:
            inv_freq, interleaved, rot_dim = self._zeros_freq(D), False, D
        else:
            inv_freq, interleaved, rot_dim = rotary
        if (self.dtype == torch.bfloat16 and self._tensor_core_ok(h, weight.w)
                and weight.n_out == (n_heads + (2 * Kh if view.writes else 0)) * D
                and self.lib.raw("rb_gemm_tc_qkv_supports")(T, D, splits)):
            q = torch.empty((T, n_heads, D), dtype=self.dtype, device=self.device)
            if pending is not None:
                self._pending_norm(pending)
            self.lib.call("rb_gemm_tc_qkv", _ptr(q), _ptr(h), h.stride(0), T, _ptr(weight.w), weight.w.stride(0), K,
                          splits, _ptr(inv_freq), _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(view.k), _ptr(view.v),
                          _ptr(view.page_table), view.max_pages, view.page_size, n_heads, Kh, D,
                          1 if view.writes else 0, 1 if interleaved else 0, rot_dim, self._stream())
            return q
        return self.rotate_append(self.linear(pending if pending is not None else h, weight), rotary, meta, view, n_heads)

    def _zeros_freq(self, D):
        z = getattr(self, "_zf", None)
        if z is None or z.shape[0] < D // 2:
            self._zf = z = torch.zeros(max(D // 2, 1), dtype=torch.float32, device=self.device)
        return z

    def attention(self, q: torch.Tensor, meta, view, n_heads: int, scale: float,
                  window: Optional[int]) -> torch.Tensor:
        """Each new token's queries over its sequence's cached keys up to its own position."""
        T, H, D = q.shape
        Kh = view.n_kv_heads
        out = torch.empty((T, H * D), dtype=self.dtype, device=self.device)
        win = int(window or 0)
        if self.dtype == torch.bfloat16 and meta.single_token and \
                self.lib.raw("rb_attention_tiled_supports")(H, Kh, D, view.page_size, 1):
            on_tma = self.decode_on_tma and self.lib.raw("rb_attention_decode_tma_supports")(H, Kh, D, view.page_size)
            if on_tma:
                n_splits = self.lib.raw("rb_attention_decode_tma_parts")(T * Kh, max(1, -(-meta.max_context // 64)), D)
            else:
                n_splits = self.lib.raw("rb_attention_decode_parts")(T, Kh, meta.max_context)
            part_o = part_ml = None
            # the parts of a small grid are a thread-block cluster and merge on chip
            on_chip = on_tma and bool(self.lib.raw("rb_attention_decode_tma_on_chip")(T * Kh, n_splits, D))
            if n_splits > 1 and not on_chip:
                part_o = torch.empty((T, H, n_splits, D), dtype=torch.float32, device=self.device)
                part_ml = torch.empty((T, H, n_splits, 2), dtype=torch.float32, device=self.device)
            if on_tma:
                # keys and values by TMA (head sizes 64 and 128)
                self.lib.call("rb_attention_decode_tma", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                              view.k.shape[0], _ptr(view.page_table), view.max_pages, view.page_size,
                              _ptr(meta.tok_pos), _ptr(meta.tok_slot), T, H, Kh, D, float(scale), win,
                              _ptr(part_o), _ptr(part_ml), n_splits, self._stream(),
                              launches=2 if n_splits > 1 and not on_chip else 1)
            else:
                self.lib.call("rb_attention_decode", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                              _ptr(view.page_table), view.max_pages, view.page_size, _ptr(meta.tok_pos),
                              _ptr(meta.tok_slot), T, H, Kh, D, float(scale), win, _ptr(part_o), _ptr(part_ml),
                              n_splits, self._stream(), launches=2 if n_splits > 1 else 1)
        elif self.dtype == torch.bfloat16 and self.prefill_on_tcgen05 and \
                self.lib.raw("rb_attention_prefill_tc_supports")(H, Kh, D, view.page_size):
            tok0, ntok, n_tiles = self._prefill_tiles(meta, 128 // (H // Kh))
            self.lib.call("rb_attention_prefill_tc", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                          view.k.shape[0], _ptr(view.page_table), view.max_pages, view.page_size,
                          _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(tok0), _ptr(ntok), n_tiles, H, Kh, D,
                          float(scale), win, self._stream())
        elif self.dtype == torch.bfloat16 and \
                self.lib.raw("rb_attention_tiled_supports")(H, Kh, D, view.page_size, 0):
            tok0, ntok, n_tiles = self._prefill_tiles(meta, 64 // (H // Kh))
            self.lib.call("rb_attention_prefill", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                          _ptr(view.page_table), view.max_pages, view.page_size, _ptr(meta.tok_pos),
                          _ptr(meta.tok_slot), _ptr(tok0), _ptr(ntok), n_tiles, H, Kh, D, float(scale), win,
                          self._stream())
        else:
            self.lib.call("rb_attention_simple", _ptr(out), _ptr(q), self.code, _ptr(view.k), _ptr(view.v),
                          _ptr(view.page_table), view.max_pages, view.page_size, _ptr(meta.tok_pos),
                          _ptr(meta.tok_slot), T, H, Kh, D, float(scale), win, self._stream())
        return out

    def _prefill_tiles(self, meta, tokens_per_tile: int):
        """Tiles of at most ``tokens_per_tile`` consecutive tokens of one sequence (device int32 arrays);
        made once per step and kept on the step's meta."""
        import numpy as np
        key = ("attention_tiles", tokens_per_tile)
        if key not in meta.extra and meta.single_token:
            # one token per sequence: a tile per row, made on the device (this also runs while a
            # decode step is being captured, where a copy from the host is not allowed)
            n = meta.n_tokens
            meta.extra[key] = (torch.arange(n, dtype=torch.int32, device=self.device),
                               torch.ones(n, dtype=torch.int32, device=self.device), n)
        if key not in meta.extra:
            tok0, ntok = [], []
            for c in meta.seqs:
                for i in range(0, c.n_new, tokens_per_tile):
                    tok0.append(c.offset + i)
                    ntok.append(min(tokens_per_tile, c.n_new - i))
            dev = torch.from_numpy(np.asarray([tok0, ntok], dtype=np.int32)).to(self.device)
            meta.extra[key] = (dev[0], dev[1], len(tok0))
        return meta.extra[key]

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        R, E = rows.shape[0], x.shape[1]
        out = torch.empty((R, E), dtype=torch.float32, device=self.device)
        self.lib.call("rb_gather_rows", _ptr(out), _ptr(x), _ptr(rows), R, E, self._stream())
        return out

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token id per row of float32 logits (into ``out`` if given); temperature <= 0 is the arg-max."""
        self._check(logits, torch.float32, "sample logits")
        R, V = logits.shape
        if out is None:
            out = torch.empty((R,), dtype=torch.int32, device=self.device)
        stats = torch.empty((R, self.lib.raw("rb_sample_chunks")(V) * 3), dtype=torch.float32, device=self.device)
        self.lib.call("rb_sample", _ptr(out), _ptr(logits), logits.stride(0), R, V, _ptr(temperature),
                      _ptr(uniform), _ptr(stats), self._stream(), launches=2)
        return out

    def decode_advance(self, token_ids: torch.Tensor, tok_pos: torch.Tensor, sampled: torch.Tensor,
                       flag_out: Optional[torch.Tensor] = None, n_live: Optional[torch.Tensor] = None) -> None:
        """token_ids <- sampled; tok_pos += 1 (the next decode step's inputs, made on the device), for the
        first ``n_live[0]`` rows (a device int32; all rows if None).
        With ``flag_out`` (one int32) the kernels' error word is written there too, so that it comes
        back with the step's results (0: no bounded wait ran out)."""
        if self._flag_ptrs is None:
            import ctypes
            a, b = ctypes.c_void_p(0), ctypes.c_void_p(0)
            self.lib.call("rb_error_flag_addresses", ctypes.byref(a), ctypes.byref(b), launches=0)
            self._flag_ptrs = (a, b)
        a, b = self._flag_ptrs if flag_out is not None else (c_void_p(0), c_void_p(0))
        self.lib.call("rb_decode_advance", _ptr(token_ids), _ptr(tok_pos), _ptr(sampled), token_ids.shape[0],
                      _ptr(n_live), a, b, _ptr(flag_out), self._stream())
