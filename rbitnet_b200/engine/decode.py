"""A decode step captured as a CUDA graph: one token for each of B sequences, sampled on
the device.

A decode step is a chain of some hundred small kernels; launched one by one from the
host, the gaps between them cost as much as the kernels.  The chain is therefore
captured once per batch size and replayed.  Which sequences, tokens and positions a
replay works on is data in fixed device buffers (slot ids index the cache's page
tables), so one graph serves any B sequences.  Per step the host writes one small
pinned buffer, copies it, replays, and reads B sampled ids back, and with them the word in
which a kernel records that one of its bounded waits ran out.

A replay also leaves the next step's inputs on the device (the sampled ids as tokens, the
positions moved on by one), so the step after it can be launched before its ids have been
read: ``launch(..., tokens=None)`` copies only that step's uniform numbers.  Host staging
buffers and result buffers are rings of four, of which at most two launches are ever outstanding.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .step import SeqChunk, StepContext, StepMeta


class DecodeGraph:
    def __init__(self, model, cache, ops, batch: int):
        self.model, self.cache, self.ops, self.B = model, cache, ops, batch
        B, dev = batch, ops.device
        # [tokens | positions | slots | wanted rows | temperatures | rows that are sequences | uniforms] as one
        # int32 buffer; the uniforms come last so that they can be copied alone
        self.RING = 4
        n = 6 * B + 1
        self.buf = torch.zeros(n, dtype=torch.int32, device=dev)
        self.hosts = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        for h in self.hosts:
            h.numpy()[3 * B:4 * B] = np.arange(B, dtype=np.int32)
        self.host = self.hosts[0]
        self.token_ids, self.tok_pos, self.tok_slot, self.want = (self.buf[i * B:(i + 1) * B] for i in range(4))
        fl = self.buf.view(torch.float32)
        self.temps, self.uniforms = fl[4 * B:5 * B], fl[5 * B + 1:6 * B + 1]
        self.n_live = self.buf[5 * B:5 * B + 1]
        self.out_hosts = [torch.zeros(B + 1, dtype=torch.int32).pin_memory() for _ in range(self.RING)]   # ids, error word
        self.out_host = self.out_hosts[0]
        self.events = [torch.cuda.Event() for _ in range(self.RING)]
        self.launched = 0
        self.result = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        self.error_code = 0
        self.meta = StepMeta(self.token_ids, self.tok_pos, self.tok_slot, self.want, B, B,
                             [SeqChunk(0, 0, 1, i) for i in range(B)], True, cache.max_seq)
        self.meta.want_every_row = True     # the wanted rows are 0 .. B-1, always
        self.graph = None
        self.sampled = None
        #: float32 logits [B, vocab] of the last replay (the graph's own buffer: copy what is to be kept)
        self.logits = None
        self.kernels = 0

    def _body(self):
        logits = self.logits = self.model.forward(StepContext(self.ops, self.meta, self.cache))
        sampled = self.ops.sample(logits, self.temps, self.uniforms, out=self.result[:self.B])
        self.ops.decode_advance(self.token_ids, self.tok_pos, sampled, flag_out=self.result[self.B:], n_live=self.n_live)
        return sampled

    def capture(self, pool=None):
        """The buffers must hold a valid step (live slots with reserved room) while this runs:
        the step is executed once for real before it is recorded."""
        keep = self.buf.clone()
        # the trial run below must leave no trace: appending keys and values again is harmless,
        # but per-sequence state would be advanced twice
        states = {e: st.clone() for e, st in self.cache.states.items()}
        side = torch.cuda.Stream(device=self.ops.device)
        side.wait_stream(torch.cuda.current_stream(self.ops.device))
        with torch.cuda.stream(side):
            self._body()
        torch.cuda.current_stream(self.ops.device).wait_stream(side)
        self.buf.copy_(keep)
        for e, st in states.items():
            self.cache.states[e].copy_(st)
        before = self.ops.lib.launches
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=pool):
            self.sampled = self._body()
        self.kernels = self.ops.lib.launches - before
        self.buf.copy_(keep)
        return self

    # ---- one step, host tokens in, host ids out
    def stage(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int],
              temperatures: Sequence[float], uniforms: Sequence[float], n_live: int = -1) -> None:
        """Every input of a step, from the host.  ``n_live``: the first so many rows are sequences that
        go on after the step (the rest belong to the padding sequence); -1: all of them."""
        B = self.B
        self.host = self.hosts[self.launched % self.RING]
        h = self.host.numpy()
        f = h.view(np.float32)
        h[0:B] = tokens
        h[B:2 * B] = positions
        h[2 * B:3 * B] = slots
        f[4 * B:5 * B] = temperatures
        h[5 * B] = B if n_live < 0 else n_live
        f[5 * B + 1:6 * B + 1] = uniforms
        self.buf.copy_(self.host, non_blocking=True)

    def stage_uniforms(self, uniforms: Sequence[float]) -> None:
        """Only a step's uniform numbers: its tokens and positions are what the step before left on the device."""
        B = self.B
        self.host = self.hosts[self.launched % self.RING]
        f = self.host.numpy().view(np.float32)
        f[5 * B + 1:6 * B + 1] = uniforms
        self.buf[5 * B + 1:6 * B + 1].copy_(self.host[5 * B + 1:6 * B + 1], non_blocking=True)

    def replay(self) -> None:
        self.graph.replay()
        self.ops.lib.launches += self.kernels

    def launch(self) -> int:
        """Replays the staged step and asks for its results; returns the ticket to ``fetch`` them with."""
        self.replay()
        ticket = self.launched
        i = ticket % self.RING
        self.out_hosts[i].copy_(self.result, non_blocking=True)
        self.events[i].record(torch.cuda.current_stream(self.ops.device))
        self.launched += 1
        return ticket

    def fetch(self, ticket: int) -> List[int]:
        """The sampled ids of launch ``ticket`` (one of the last two); ``error_code`` is the kernels' error word."""
        if not self.launched - 2 <= ticket < self.launched:
            raise ValueError(f"launch {ticket} is not among the last two of {self.launched}")
        i = ticket % self.RING
        self.events[i].synchronize()
        out = self.out_hosts[i].tolist()
        self.error_code = out[self.B]
        return out[:self.B]

    def read(self) -> List[int]:
        """The sampled ids of the last replay made with ``replay()``; ``error_code`` is the kernels' error word (0: none)."""
        self.out_host.copy_(self.result, non_blocking=True)
        torch.cuda.current_stream(self.ops.device).synchronize()
        out = self.out_host.tolist()
        self.error_code = out[self.B]
        return out[:self.B]

    @property
    def h2d_bytes(self) -> int:
        return self.host.numel() * 4

    @property
    def d2h_bytes(self) -> int:
        return self.out_host.numel() * 4
