"""Engine: the entry point a program uses.  A model folder (or a configuration and a
seed) in, token ids out.

It keeps the reference façade's names where the reference has them
(crates/bitnet-core/src/inference.rs:75-209): ``Engine.load_path``,
``Engine.from_env`` (RBITNET_MODEL, and RBITNET_TOY / RBITNET_TOY_SEED for
seeded random weights without a file), ``complete(prompt, max_tokens,
temperature)``, ``is_ready``, ``model_summary``, ``tensor_count``,
``tensor_names_preview``.  ``generate`` is the batched, ids-in ids-out call the
reference lacks.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache import SequenceCache, PAGE_SIZE
from ..config import ModelConfig, load_config, get_architecture, config_from_dict, ConfigError
from ..weights import read_model_tensors, random_tensors
from .generate import GenerationLoop, GenerationResult
from .model import Model
from .step import Stepper, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


class TokenizerMissing(RuntimeError):
    """``complete`` needs tokenizer.json beside the model, or RBITNET_TOKENIZER
    (crates/bitnet-core/src/inference.rs:55-71)."""


def _dtype(d):
    if isinstance(d, torch.dtype):
        return d
    if d not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, found {d!r}")
    return _DTYPES[d]


def _no_parent_components(path) -> None:
    # crates/bitnet-core/src/inference.rs:44-53
    if ".." in Path(path).parts:
        raise ValueError("path must not contain '..' components")


class Engine:
    def __init__(self, config: ModelConfig, tensors: Dict[str, torch.Tensor], dtype="bfloat16",
                 device="cuda:0", max_tokens: Optional[int] = None, max_seq: Optional[int] = None,
                 max_batch: int = 64, page_size: int = PAGE_SIZE, max_batch_tokens: int = 8192,
                 ops=None, model_path: Optional[Path] = None, verbose: bool = False,
                 use_graphs: bool = True):
        """max_seq: longest sequence (default: the configuration's max positions).
        max_tokens: cache size in positions over all live sequences, each rounded up to
        whole pages (default: max_batch sequences of max_seq)."""
        from ..kernels.ops import CudaOps
        self.config = config
        self.model_path = model_path
        self.dtype = _dtype(dtype)
        self.ops = ops if ops is not None else CudaOps(self.dtype, device, verbose_build=verbose)
        self.spec = get_architecture(config.architecture).build_spec(config)
        self._tensor_names = sorted(tensors)
        self.model = Model(self.spec, tensors, self.ops)
        self.max_seq = int(max_seq or self.spec.max_positions)
        if self.max_seq > self.spec.max_positions:
            raise ValueError(f"max_seq {self.max_seq} exceeds the model's max positions "
                             f"{self.spec.max_positions}")
        self.max_batch = max_batch
        if max_tokens is None:
            max_tokens = max_batch * (-(-self.max_seq // page_size) * page_size)
        #: decode steps run as captured CUDA graphs (one per batch size)
        self.use_graphs = use_graphs and ops is None
        cache_needs, reads, state_needs = self.model.cache_plan()
        # The captured step of a batch size between two graphs is filled up with rows of a padding
        # sequence.  It gets a slot and a page of its own, beyond what the caller asked for, here and
        # now: taken at its first use it could take a page that a running batch was promised.
        n_pages = max(1, -(-max_tokens // page_size))
        extra = 1 if self.use_graphs else 0
        self.cache = SequenceCache(cache_needs, reads, state_needs, (n_pages + extra) * page_size, self.max_seq,
                                   self.dtype, self.ops.device, page_size=page_size, n_slots=n_pages + extra)
        self._pad_slot = None
        if self.use_graphs:
            self._pad_slot = self.cache.alloc()
            self.cache.reserve(self._pad_slot, 1)
        self.stepper = Stepper(self.model, self.cache, self.ops, max_batch_tokens=max_batch_tokens)
        self.stop_ids = list(self.spec.stop_ids)
        self._tokenizer = None
        self._graphs = {}
        self._graph_pool = None
        self._last_slots, self._last_graph = [], None

    # ------------------------------------------------------------------ construction
    @classmethod
    def load_path(cls, path, **kw) -> "Engine":
        """A model folder with config.json and model.safetensors."""
        path = Path(path)
        config = load_config(path)
        tensors = read_model_tensors(path)
        return cls(config, tensors, model_path=path, **kw)

    from_pretrained = load_path

    @classmethod
    def from_random(cls, config, seed: int = 42, **kw) -> "Engine":
        """Seeded random weights, made in memory (no file)."""
        if isinstance(config, dict):
            config = config_from_dict(config)
        spec = get_architecture(config.architecture).build_spec(config)
        dtype = _dtype(kw.get("dtype", "bfloat16"))
        dev = kw.get("device", "cuda:0") if torch.cuda.is_available() and kw.get("ops") is None else "cpu"
        tensors = random_tensors(spec, seed, dtype=dtype, device=dev)
        return cls(config, tensors, **kw)

    @classmethod
    def from_env(cls, **kw) -> "Engine":
        """RBITNET_MODEL: a model folder.  Else RBITNET_TOY=1 with RBITNET_TOY_CONFIG
        (a config.json) and RBITNET_TOY_SEED (default 42): random weights."""
        path = os.environ.get("RBITNET_MODEL")
        if path:
            _no_parent_components(path)
            return cls.load_path(path, **kw)
        if os.environ.get("RBITNET_TOY") in ("1", "true", "yes"):
            cfg_path = os.environ.get("RBITNET_TOY_CONFIG")
            if not cfg_path:
                raise ConfigError("RBITNET_TOY needs RBITNET_TOY_CONFIG, the config.json to draw weights for")
            _no_parent_components(cfg_path)
            import json
            seed = int(os.environ.get("RBITNET_TOY_SEED", "42"))
            return cls.from_random(json.loads(Path(cfg_path).read_text()), seed, **kw)
        raise ConfigError("model not loaded: set RBITNET_MODEL (or RBITNET_TOY and RBITNET_TOY_CONFIG)")

    # ------------------------------------------------------------------ information
    def is_ready(self) -> bool:
        return True

    def tensor_count(self) -> int:
        return len(self._tensor_names)

    def tensor_names_preview(self, max_names: int) -> List[str]:
        return self._tensor_names[:max_names]

    def model_summary(self) -> str:
        c = self.config
        n = sum(int(np.prod(s)) for s in self.spec.expected_shapes().values())
        return (f"{c.architecture} layers={len(self.spec.layers)} width={self.spec.width} "
                f"vocab={self.spec.vocab_size} params={n} dtype={str(self.dtype).replace('torch.', '')} "
                f"cache={self.cache.bytes() / 2**20:.1f}MiB")

    # ------------------------------------------------------------------ stepping
    def live_sequences(self) -> List[int]:
        """Slots held by callers (the engine's own padding sequence is not counted)."""
        return [s for s in self.cache.book.live() if s != self._pad_slot]

    def new_sequence(self) -> int:
        return self.cache.alloc()

    def end_sequence(self, slot: int) -> None:
        self.cache.free(slot)

    def step(self, entries: Sequence[StepEntry], captured: bool = False) -> Optional[torch.Tensor]:
        """Runs the entries' tokens from the cache; float32 logits [wanted places, vocab] or None.
        ``captured``: a step of one token per sequence runs as the captured decode step that
        ``generate`` uses (CUDA graph, padding rows, arg-max sampling whose ids are dropped) instead of
        kernel by kernel, so that its logits can be compared too."""
        if captured and self.use_graphs and entries and all(len(e.tokens) == 1 for e in entries):
            slots = [e.slot for e in entries]
            if len(set(slots)) != len(slots):
                raise ValueError("a slot appears twice in one step")
            V = self.model.vocab_size
            for e in entries:
                if not 0 <= int(e.tokens[0]) < V:
                    raise ValueError(f"slot {e.slot}: token id out of range (vocabulary {V})")
                if any(w != 0 for w in e.want):
                    raise ValueError(f"slot {e.slot}: wanted place is not among its 1 tokens")
            n = len(entries)
            self._decode_step([(e.slot, list(e.tokens)) for e in entries], [0.0] * n, [0.0] * n)
            rows = [i for i, e in enumerate(entries) if len(e.want)]
            if not rows:
                return None
            return self._last_graph.logits[rows].clone()
        return self.stepper.step(entries)

    def decode_graph(self, batch: int):
        """The captured decode step for ``batch`` sequences (made at first use).  Needs ``batch``
        live slots with room for one more token each at the time of the first call."""
        g = self._graphs.get(batch)
        if g is None:
            from .decode import DecodeGraph
            g = DecodeGraph(self.model, self.cache, self.ops, batch)
            self._graphs[batch] = g
        return g

    @staticmethod
    def _graph_batch(n: int) -> int:
        """Batch sizes that get a captured step of their own: 1, 2, 4, then multiples of 8."""
        return n if n <= 2 else (4 if n <= 4 else -(-n // 8) * 8)

    def _decode_launch(self, feed, temperatures, uniforms):
        """Launches one captured decode step and returns a ticket for ``_decode_fetch``.  ``feed``:
        (slot, [token]) pairs with the tokens from the host; or None: the same sequences as the launch
        before, whose tokens and positions that step left on the device (only the uniform numbers are
        copied), which is how a step is launched before the ids of the step before it have been read.
        The sequences' lengths move on at once."""
        if feed is not None:
            slots = [s for s, _ in feed]
            tokens = [t[0] for _, t in feed]
        else:
            slots = self._last_slots
        n = len(slots)
        positions = self.cache.lengths(slots)
        self.cache.reserve_one_each(slots)
        temperatures, uniforms = list(temperatures), list(uniforms)
        batch = self._graph_batch(n)
        extra = batch - n
        if extra:
            temperatures += [0.0] * extra
            uniforms += [0.0] * extra
        self.cache.upload_tables()
        g = self.decode_graph(batch)
        if feed is not None or g.graph is None:
            if feed is None:
                raise RuntimeError("a decode step without tokens needs the captured step of the launch before it")
            # rows of the padding sequence fill the step up: they rewrite its position 0 and their results are dropped
            g.stage(slots + [self._pad_slot] * extra, tokens + [0] * extra, positions + [0] * extra,
                    temperatures, uniforms, n_live=n)
            if g.graph is None:
                g.capture(pool=self._graph_pool)
                if self._graph_pool is None:
                    self._graph_pool = g.graph.pool()
        else:
            g.stage_uniforms(uniforms)
        ticket = g.launch()
        self.cache.advance_one_each(slots)
        self._last_slots, self._last_graph = slots, g
        return (g, ticket, n)

    def _decode_fetch(self, ticket) -> List[int]:
        g, t, n = ticket
        ids = g.fetch(t)[:n]
        if g.error_code:
            self.ops.check_errors()            # raises with the code, and clears the word
        return ids

    def _decode_step(self, feed, temperatures, uniforms) -> List[int]:
        return self._decode_fetch(self._decode_launch(feed, temperatures, uniforms))

    # the generation loop's names for the two halves of a decode step
    decode_launch = _decode_launch
    decode_fetch = _decode_fetch

    def _step_sample(self, feed, temperatures, uniforms) -> List[int]:
        if self.use_graphs and all(len(t) == 1 for _, t in feed):
            return self._decode_step(feed, temperatures, uniforms)   # the error word comes back with the ids
        entries = [StepEntry(slot, toks, [len(toks) - 1]) for slot, toks in feed]
        logits = self.stepper.step(entries)
        params = torch.from_numpy(np.asarray([temperatures, uniforms], dtype=np.float32)).to(self.ops.device)
        ids = self.ops.sample(logits, params[0], params[1]).tolist()
        if hasattr(self.ops, "check_errors"):
            self.ops.check_errors()
        return ids

    # ------------------------------------------------------------------ generation
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 256, temperature: float = 0.7,
                 seed: int = 0, stop_ids: Optional[Sequence[int]] = None,
                 max_batch: Optional[int] = None, on_token=None) -> List[GenerationResult]:
        """Token-id prompts in, generated ids out, one result per prompt in order.
        temperature <= 0 is greedy.  Defaults are the reference server's
        (crates/bitnet-server/src/lib.rs:317, :358).  ``on_token(request index, token id)`` is
        called for every emitted token as soon as the host has it."""
        loop = GenerationLoop(self._step_sample, self.cache, max_batch or self.max_batch,
                              decoder=self if self.use_graphs else None)
        out = loop.run(prompts, max_tokens, temperature, seed,
                       self.stop_ids if stop_ids is None else stop_ids, on_token=on_token)
        self.last_stats = {"steps": loop.steps, "prefill_tokens": loop.prefill_tokens,
                           "decode_tokens": loop.decode_tokens}
        return out

    def _load_tokenizer(self):
        if self._tokenizer is None:
            cand = os.environ.get("RBITNET_TOKENIZER")
            paths = [Path(cand)] if cand else []
            if self.model_path is not None:
                paths.append(Path(self.model_path) / "tokenizer.json")
            path = next((p for p in paths if p.is_file() and p.name == "tokenizer.json"), None)
            if path is None:
                raise TokenizerMissing("tokenizer.json not found beside the model (or set RBITNET_TOKENIZER)")
            from tokenizers import Tokenizer
            self._tokenizer = Tokenizer.from_file(str(path))
        return self._tokenizer

    def complete(self, prompt: str, max_tokens: int, temperature: float) -> str:
        """Text in, text out, as crates/bitnet-core/src/inference.rs:183-208 /
        crates/bitnet-core/src/llama/runtime.rs:34-78: encode with special tokens, stop at the
        first of "</s>", "<|endoftext|>", "<|im_end|>" the tokenizer knows, decode
        skipping special tokens."""
        tok = self._load_tokenizer()
        ids = tok.encode(prompt, add_special_tokens=True).ids
        if not ids:
            return ""
        eos = next((tok.token_to_id(t) for t in ("</s>", "<|endoftext|>", "<|im_end|>")
                    if tok.token_to_id(t) is not None), None)
        res = self.generate([ids], max_tokens, temperature, stop_ids=[] if eos is None else [eos])[0]
        return tok.decode(res.tokens, skip_special_tokens=True)
