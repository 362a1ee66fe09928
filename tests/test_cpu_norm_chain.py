"""How a block hands a norm to the products around it, on the torch stand-in (no GPU): operations that
offer ``norm_request`` get asked, parts that say ``folds_norms`` get rows with their norm pending and pass
the request for the next norm on, anything else gets normed rows from the norm itself; and the result is
the same either way."""
from dataclasses import dataclass

import pytest
import torch

from helpers import assert_close, make_model_dir, PlainModel
from tiny import TINY_A, TINY_B, prompts
from torch_ops import TorchOps


@dataclass
class _Request:
    weight: torch.Tensor
    eps: float
    result: object = None


@dataclass
class _Rows:                      # rows with their norm pending, as the CUDA operations hand them on
    x: torch.Tensor
    weight: torch.Tensor
    eps: float

    @property
    def shape(self):
        return self.x.shape


class FoldingOps(TorchOps):
    """The stand-in with a norm folded into the products around it, for at most ``up_to`` rows."""

    def __init__(self, up_to=1 << 30):
        super().__init__(torch.float32)
        self.up_to = up_to
        self.norm_kernels = self.requests = self.granted = self.pending_in = 0

    def rmsnorm(self, x, w, eps, out_dtype=None):
        self.norm_kernels += 1
        return super().rmsnorm(x, w, eps, out_dtype)

    def norm_request(self, weight, eps):
        self.requests += 1
        return _Request(weight, eps)

    def normed(self, rows):
        return self.rmsnorm(rows.x, rows.weight, rows.eps)

    def _take(self, x):
        """(input of the product, per-row factor or None)"""
        if not isinstance(x, _Rows):
            return x, None
        self.pending_in += 1
        factor = 1.0 / torch.sqrt((x.x * x.x).mean(-1, keepdim=True) + x.eps)
        return x.x * x.weight, factor

    def linear(self, x, weight, out_dtype=None, accumulate_into=None, scale=1.0, then_norm=None):
        x, factor = self._take(x)
        y = x.to(torch.float32) @ weight.w.to(torch.float32).T * scale
        if factor is not None:
            y = y * factor
        if accumulate_into is not None:
            accumulate_into += y
            if then_norm is not None and accumulate_into.shape[0] <= self.up_to:
                self.granted += 1
                then_norm.result = _Rows(accumulate_into, then_norm.weight, then_norm.eps)
            return accumulate_into
        return y.to(out_dtype or self.dtype)

    def gated_linear(self, x, weight):
        x, factor = self._take(x)
        gu = x.to(torch.float32) @ weight.w.to(torch.float32).T
        if factor is not None:
            gu = gu * factor
        g, u = gu[:, :weight.inner], gu[:, weight.inner:]
        return (g / (1.0 + torch.exp(-g)) * u).to(self.dtype)


def _engine(folder, ops):
    from rbitnet_b200 import Engine
    return Engine.load_path(folder, dtype="float32", ops=ops, max_tokens=1024, page_size=16)


@pytest.mark.parametrize("cfg,seed", [(TINY_A, 0), (TINY_B, 2)])
def test_a_norm_handed_to_the_products_around_it_changes_nothing(tmp_path, cfg, seed):
    from rbitnet_b200 import StepEntry
    folder = make_model_dir(tmp_path / "m", cfg, seed)
    ref = PlainModel(folder)
    layers = cfg["num_hidden_layers"]
    p = prompts([19], cfg["vocab_size"], 70)[0]
    for up_to, folded in ((1 << 30, True), (4, False)):
        ops = FoldingOps(up_to)
        eng = _engine(folder, ops)
        s = eng.new_sequence()
        out = eng.step([StepEntry(s, p, list(range(len(p))))])
        assert_close(out, ref.logits(p), "float32", "a prompt with its norms handed on")
        # every norm between two products is asked for; the first layer's first norm and the final norm are kernels
        assert ops.requests == 2 * layers - 1
        if folded:
            assert ops.granted == ops.pending_in == 2 * layers - 1 and ops.norm_kernels == 2
        else:                                   # 19 rows are more than the operations fold: every norm is a kernel
            assert ops.granted == ops.pending_in == 0 and ops.norm_kernels == 2 * layers + 1
        # one token: folded in both
        before = ops.norm_kernels
        out = eng.step([StepEntry(s, [5], [0])])
        assert_close(out, ref.logits(p + [5])[-1:], "float32", "one more token")
        assert ops.norm_kernels - before == 2


def test_parts_and_blocks_that_know_nothing_of_it_get_normed_rows(tmp_path):
    """A mixer without ``folds_norms`` gets a tensor and no request; a block without ``chains_norms`` is run
    with three arguments; the blocks around them go on handing norms on among themselves."""
    from rbitnet_b200.parts.registry import register_part, build_part
    from rbitnet_b200.parts.block import PreNormBlock
    from rbitnet_b200.parts.attention import Attention
    seen = []

    class PlainAttention(Attention):
        folds_norms = False

        def forward(self, ctx, h, entry, accumulate_into):          # (the signature of old: no then_norm)
            seen.append(type(h))
            return super().forward(ctx, h, entry, accumulate_into)

    class OldBlock:                      # an arrangement that knows nothing of handing norms on
        def __init__(self, spec):
            self.inner = PreNormBlock(spec)
            self.mixer = self.inner.mixer

        def parts(self):
            return self.inner.parts()

        def run(self, ctx, x, entry):
            assert self.inner.run(ctx, x, entry) is None

    register_part("mixer", "plain_attention_for_test", PlainAttention)
    register_part("block", "old_block_for_test", OldBlock)
    from rbitnet_b200.config import config_from_dict
    from rbitnet_b200.config.registry import get_architecture
    from rbitnet_b200.weights import random_tensors
    from rbitnet_b200.engine.model import Model
    from rbitnet_b200.cache import SequenceCache
    import numpy as np
    from rbitnet_b200.engine.step import SeqChunk, StepContext, build_meta
    cfg = config_from_dict(TINY_B)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    assert len(spec.layers) >= 3
    tensors = random_tensors(spec, 5)
    spec.layers[1].parts["mixer"].kind = "plain_attention_for_test"
    spec.layers[2].arrangement = "old_block_for_test"

    def run(ops):
        model = Model(spec, tensors, ops)
        needs, reads, states = model.cache_plan()
        cache = SequenceCache(needs, reads, states, max_tokens=128, max_seq=128, dtype=torch.float32, device=ops.device,
                              page_size=16)
        s = cache.alloc()
        T = 6
        cache.reserve(s, T)
        cache.upload_tables()
        ids = np.arange(3, 3 + T, dtype=np.int32)
        meta = build_meta([SeqChunk(s, 0, T, 0)], ids, np.arange(T, dtype=np.int32), ops.device)
        return model.forward(StepContext(ops, meta, cache))

    folding = FoldingOps()
    got = run(folding)
    want = run(TorchOps(torch.float32))
    assert_close(got, want, "float32", "mixed blocks")
    assert seen and all(t is torch.Tensor for t in seen)
    assert len(spec.layers) == 3
    # Layer 0 hands its second norm on and leaves layer 1's first (2 granted, 1 taken); layer 1's mixer takes
    # no pending rows, so what was left for it is normed by the norm's kernel, and it is asked for nothing, so
    # its second norm is a kernel too; layer 2 is an old block: nobody leaves it rows or asks it for more, and
    # inside it the second norm is handed on (1 granted, 1 taken).  Kernels: layer 0's first norm, layer 1's
    # two, layer 2's first, the final norm.
    assert (folding.granted, folding.pending_in, folding.norm_kernels) == (3, 2, 5)
