"""The generation loop above the step function.

Requests (token-id lists of unequal lengths) are taken in order into batches.
A batch's prompts run in one step, then every live sequence advances one token
per step.  A sampled stop token ends its sequence and is not emitted; a
sequence also ends at ``max_tokens`` new tokens or when it has reached the
longest length the cache holds.  A sequence that has ended leaves the batch and
gives its slot back at once; the next batch uses the slots again.  No step runs
after the last wanted token that could have been known to be the last.

With a ``decoder`` (an engine whose decode steps are captured and leave the next
step's inputs on the device) the loop launches step k+1 before it has read the ids
of step k, whenever no sequence of step k can end by length: the device then never
waits for the host's bookkeeping.  If a sequence does sample a stop token at step k,
its part of step k+1 is dropped (its slot is already given back; what that step
wrote there is never read) and the other sequences' ids of step k+1 stand: a
sequence's result does not depend on what else was in its batch.

The reference's loop handles one prompt: prompt token by token, then sample,
append, forward until max_tokens or EOS
(crates/bitnet-core/src/llama/runtime.rs:34-78; EOS not emitted :67-69; empty
prompt gives an empty result :46-48).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.rng import uniforms


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str          # "stop" | "length" | "empty"
    prompt_tokens: int


@dataclass
class _Live:
    request: int
    slot: int
    last: int
    out: List[int] = field(default_factory=list)


class GenerationLoop:
    """``step_sample(entries, temperatures, uniforms) -> list of token ids`` runs one step
    over ``(slot, tokens)`` pairs and samples at each sequence's last token.  ``cache``
    provides ``alloc() -> slot``, ``free(slot)``, ``length(slot)``, ``max_seq`` and
    ``fits(lengths, prompts) -> bool`` (whether sequences whose prompts of these sizes grow to
    these lengths fit together)."""

    def __init__(self, step_sample: Callable, cache, max_batch: int, decoder=None):
        """``decoder``: None, or an object with ``decode_launch(feed | None, temperatures, uniforms) ->
        ticket`` (feed None: the sequences of the launch before, their tokens taken from that step on
        the device; lengths in ``cache`` move on at once) and ``decode_fetch(ticket) -> ids``."""
        self.step_sample, self.cache, self.max_batch = step_sample, cache, max_batch
        self.decoder = decoder
        self.steps = 0
        self.prefill_tokens = 0
        self.decode_tokens = 0

    def _take_batch(self, pending: List[int], prompts, max_tokens: int) -> List[int]:
        batch: List[int] = []
        lengths: List[int] = []
        firsts: List[int] = []
        for r in pending:
            if len(batch) >= self.max_batch:
                break
            n = len(prompts[r])
            if n > self.cache.max_seq:
                raise ValueError(f"request {r}: prompt of {n} tokens exceeds the longest sequence "
                                 f"the cache holds ({self.cache.max_seq})")
            grown = min(n + max_tokens, self.cache.max_seq)
            if not self.cache.fits(lengths + [grown], firsts + [n]):
                break
            batch.append(r)
            lengths.append(grown)
            firsts.append(n)
        if not batch:
            raise ValueError(f"request {pending[0]} does not fit the cache even alone")
        return batch

    def run(self, prompts: Sequence[Sequence[int]], max_tokens: int, temperature: float = 0.0,
            seed: int = 0, stop_ids: Sequence[int] = (),
            on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        stop = set(int(s) for s in stop_ids)
        results: List[Optional[GenerationResult]] = [None] * len(prompts)
        pending = []
        for r, p in enumerate(prompts):
            if len(p) == 0:
                results[r] = GenerationResult([], "empty", 0)
            elif max_tokens <= 0:
                results[r] = GenerationResult([], "length", len(p))
            else:
                pending.append(r)
        def draws(seqs, ahead=0):
            if temperature > 0:              # a draw per request, a function of (seed, request, tokens so far)
                return uniforms(seed, [s.request for s in seqs], [len(s.out) + ahead for s in seqs]).tolist()
            return [0.0] * len(seqs)         # the arg-max needs none

        def take(seqs, sampled, fed_ahead=0):
            """Books one sampled token per sequence; returns the sequences that go on.  ``fed_ahead``: steps
            launched after the one these tokens come from, which the cache's lengths already count."""
            still: List[_Live] = []
            for s, tok in zip(seqs, sampled):
                tok = int(tok)
                reason = None
                if tok in stop:
                    reason = "stop"
                else:
                    s.out.append(tok)
                    s.last = tok
                    if on_token is not None:
                        on_token(s.request, tok)
                    if len(s.out) >= max_tokens:
                        reason = "length"
                    elif self.cache.length(s.slot) - fed_ahead >= self.cache.max_seq:
                        reason = "length"       # no room to feed this token back
                if reason is None:
                    still.append(s)
                else:
                    results[s.request] = GenerationResult(s.out, reason, len(prompts[s.request]))
                    self.cache.free(s.slot)
                    s.slot = -1
            return still

        while pending:
            batch = self._take_batch(pending, prompts, max_tokens)
            pending = pending[len(batch):]
            live = [_Live(r, self.cache.alloc(), -1) for r in batch]
            try:
                feed = [(s.slot, list(prompts[s.request])) for s in live]
                self.prefill_tokens += sum(len(t) for _, t in feed)
                if self.decoder is not None:
                    # the prompts in one step, then decode steps launched ahead of their results
                    live = take(live, self.step_sample(feed, [temperature] * len(live), draws(live)))
                    self.steps += 1
                    while live:
                        temps = [temperature] * len(live)
                        self.decode_tokens += len(live)
                        ticket = self.decoder.decode_launch([(s.slot, [s.last]) for s in live], temps, draws(live))
                        flying = live                     # the sequences of the launch whose ids come next
                        while True:
                            ahead = None
                            # Every sequence of the step in flight goes on after it unless it samples a stop
                            # token (its lengths already count that step): the next step can be launched now.
                            if all(len(s.out) + 1 < max_tokens and self.cache.length(s.slot) < self.cache.max_seq
                                   for s in flying):
                                ahead = self.decoder.decode_launch(None, temps, draws(flying, ahead=1))
                            live = take(flying, self.decoder.decode_fetch(ticket), fed_ahead=0 if ahead is None else 1)
                            self.steps += 1
                            if ahead is None:
                                break
                            if len(live) == len(flying):  # nobody left: the step launched ahead is the step in flight
                                ticket = ahead
                                self.decode_tokens += len(live)
                                continue
                            # somebody left: the step launched ahead still holds the others' next tokens
                            ids = self.decoder.decode_fetch(ahead)
                            if live:
                                self.decode_tokens += len(live)
                                self.steps += 1
                                live = take(live, [i for s, i in zip(flying, ids) if s.slot >= 0])
                            break
                    continue
                while live:
                    sampled = self.step_sample(feed, [temperature] * len(live), draws(live))
                    self.steps += 1
                    live = take(live, sampled)
                    feed = [(s.slot, [s.last]) for s in live]
                    self.decode_tokens += len(live)
            finally:
                for s in live:
                    if s.slot >= 0:
                        self.cache.free(s.slot)
        return results  # type: ignore[return-value]
