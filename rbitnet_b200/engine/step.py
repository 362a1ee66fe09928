"""The step function: runs the tokens it is given, as one batch, from the cache, and
returns the logits at the wanted places.

A step holds, for each of its sequences, the sequence's next tokens (its whole
prompt, or one token, or any number) and the places among them whose logits
are wanted.  Positions are implied by the cache: a sequence's new tokens sit at
``length .. length + n - 1``.  All sequences' tokens are packed into one batch
of rows without padding, so padding cannot change a result.  The reference's
equivalent handles one token of one sequence per call
(crates/bitnet-core/src/llama/model.rs:219-227 for its guards: position below
the maximum, token id inside the vocabulary).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    #: indices into ``tokens`` whose logits are wanted (may be empty)
    want: Sequence[int] = ()


@dataclass
class SeqChunk:
    """The part of one sequence that a batch of rows holds."""
    slot: int
    start: int      # position of its first row in the sequence
    n_new: int
    offset: int     # index of its first row in the batch


@dataclass
class StepMeta:
    """Where each row of the batch belongs, on the device (int32) and on the host."""
    token_ids: torch.Tensor
    tok_pos: torch.Tensor
    tok_slot: torch.Tensor
    want_rows: torch.Tensor
    n_tokens: int
    n_want: int
    seqs: List[SeqChunk]
    single_token: bool              # every sequence brings exactly one token
    max_context: int                # longest sequence length after this batch
    extra: dict = field(default_factory=dict)
    want_every_row: bool = False    # want_rows is 0, 1, .., n_tokens-1: the rows need no gathering


class StepContext:
    def __init__(self, ops, meta: StepMeta, cache):
        self.ops, self.meta, self.cache = ops, meta, cache

    def cache_view(self, entry: int):
        return self.cache.view(entry)

    def state_view(self, entry: int):
        return self.cache.state(entry)


def build_meta(chunks: List[SeqChunk], tokens: np.ndarray, want_rows: np.ndarray, device) -> StepMeta:
    T = int(tokens.shape[0])
    pos = np.empty(T, dtype=np.int32)
    slot = np.empty(T, dtype=np.int32)
    for c in chunks:
        pos[c.offset:c.offset + c.n_new] = np.arange(c.start, c.start + c.n_new, dtype=np.int32)
        slot[c.offset:c.offset + c.n_new] = c.slot
    R = int(want_rows.shape[0])
    packed = np.concatenate([tokens.astype(np.int32), pos, slot, want_rows.astype(np.int32)])
    dev = torch.from_numpy(packed).to(device)       # pageable copy: staged before the call returns
    meta = StepMeta(dev[0:T], dev[T:2 * T], dev[2 * T:3 * T], dev[3 * T:3 * T + R], T, R, chunks,
                    all(c.n_new == 1 for c in chunks),
                    max((c.start + c.n_new for c in chunks), default=0))
    meta.want_every_row = R == T and bool(np.array_equal(want_rows, np.arange(T)))
    return meta


class Stepper:
    def __init__(self, model, cache, ops, max_batch_tokens: int = 8192):
        self.model, self.cache, self.ops = model, cache, ops
        self.max_batch_tokens = max_batch_tokens

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Returns float32 logits [number of wanted places, vocab] on the device, in the
        order of the entries and of each entry's ``want``; None if nothing is wanted."""
        V = self.model.vocab_size
        seen = set()
        for e in entries:
            if len(e.tokens) < 1:
                raise ValueError(f"slot {e.slot}: a step needs at least one token per sequence")
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            toks = np.asarray(e.tokens)
            if toks.min() < 0 or toks.max() >= V:
                raise ValueError(f"slot {e.slot}: token id out of range (vocabulary {V})")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"slot {e.slot}: wanted place {w} is not among its {len(e.tokens)} tokens")
        for e in entries:
            self.cache.reserve(e.slot, len(e.tokens))
        self.cache.upload_tables()

        # rows of the whole step, then cut into batches of at most max_batch_tokens rows
        outputs = []
        batch: List[SeqChunk] = []
        batch_tokens: List[np.ndarray] = []
        batch_want: List[int] = []
        rows = 0

        def flush():
            nonlocal batch, batch_tokens, batch_want, rows
            if not batch:
                return
            meta = build_meta(batch, np.concatenate(batch_tokens), np.asarray(batch_want, dtype=np.int32),
                              self.ops.device)
            out = self.model.forward(StepContext(self.ops, meta, self.cache))
            if out is not None:
                outputs.append(out)
            batch, batch_tokens, batch_want, rows = [], [], [], 0

        for e in entries:
            toks = np.asarray(e.tokens, dtype=np.int32)
            base = self.cache.length(e.slot)
            want = sorted(e.want)
            if list(want) != list(e.want):
                raise ValueError(f"slot {e.slot}: wanted places must be ascending")
            done = 0
            while done < len(toks):
                room = self.max_batch_tokens - rows
                if room == 0:
                    flush()
                    room = self.max_batch_tokens
                n = min(room, len(toks) - done)
                batch.append(SeqChunk(e.slot, base + done, n, rows))
                batch_tokens.append(toks[done:done + n])
                batch_want.extend(rows + (w - done) for w in want if done <= w < done + n)
                rows += n
                done += n
        flush()
        for e in entries:
            self.cache.advance(e.slot, len(e.tokens))
        if not outputs:
            return None
        return outputs[0] if len(outputs) == 1 else torch.cat(outputs, dim=0)
