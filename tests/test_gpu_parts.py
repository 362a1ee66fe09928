"""Each part of a layer alone against the plain implementation's function for it, and the
generality of the way layers are put together: a schedule that names a layer twice and lets a
run read another run's cache, a window, and a toy mixer with state of its own that is defined
here, registered, built and stepped without touching the package's files."""
import json
import math
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

import plain_llama as plain
from helpers import assert_close, make_model_dir, PlainModel, sharpen, TOL
from tiny import TINY_A, TINY_B, prompts

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _ops(dtype):
    from rbitnet_b200.kernels.ops import CudaOps
    return CudaOps(DTYPES[dtype])


def _ctx(ops, cache, chunks):
    """A step context for chunks [(slot, start, n_new)] packed in order."""
    import numpy as np
    from rbitnet_b200.engine.step import SeqChunk, StepContext, build_meta
    seqs, off = [], 0
    for slot, start, n in chunks:
        seqs.append(SeqChunk(slot, start, n, off))
        off += n
    meta = build_meta(seqs, np.zeros(off, dtype=np.int32), np.zeros(0, dtype=np.int32), ops.device)
    return StepContext(ops, meta, cache)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,eps", [(48, 1e-5), (272, 1e-6)])
def test_norm_part(dtype, width, eps):
    from rbitnet_b200.parts import build_part, PartSpec
    ops = _ops(dtype)
    part = build_part("norm", PartSpec("rmsnorm", {"width": width, "eps": eps}))
    torch.manual_seed(51)
    assert part.weight_shapes() == {"weight": ((width,), "norm")}
    w = 1 + 0.1 * torch.randn(width)
    part.bind({"weight": w.to(DTYPES[dtype]).cuda()}, ops)
    x = torch.randn(7, width) * 2
    got = part.forward(_ctx(ops, None, [(0, 0, 7)]), x.cuda())
    ref = plain.rmsnorm(x.double(), w.to(DTYPES[dtype]).double(), eps)
    assert_close(got, ref, dtype, "rmsnorm part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from rbitnet_b200.parts import build_part, PartSpec
    ops = _ops(dtype)
    E, F, T = 72, 200, 9
    torch.manual_seed(52)
    part = build_part("feed_forward", PartSpec("gated_dense", {"width": E, "inner": F, "activation": "silu"}))
    dt = DTYPES[dtype]
    w = {"gate": (torch.randn(F, E) / 6).to(dt), "up": (torch.randn(F, E) / 6).to(dt), "down": (torch.randn(E, F) / 10).to(dt)}
    part.bind({k: v.cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E).to(dt)
    resid = torch.randn(T, E)
    x = resid.clone().cuda()
    part.forward(_ctx(ops, None, [(0, 0, T)]), h.cuda(), accumulate_into=x)
    ref = resid.double() + plain.gated_mlp(h.double(), {k: v.double() for k, v in w.items()})
    assert_close(x, ref, dtype, "gated feed-forward part")
    with pytest.raises(ValueError, match="activation"):
        build_part("feed_forward", PartSpec("gated_dense", {"width": 8, "inner": 8, "activation": "relu"}))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,K,D,pairing,theta,window,scale", [(4, 2, 16, "interleaved", 1e4, None, None),
                                                             (3, 1, 32, "half", 5e5, 6, 0.3),
                                                             (6, 3, 48, "half", 1e4, None, None)])
def test_attention_mixer_part_in_steps(dtype, H, K, D, pairing, theta, window, scale):
    """The mixer alone over a cache: two sequences, a prompt chunk each, then single tokens."""
    from rbitnet_b200.parts import build_part, PartSpec
    from rbitnet_b200.cache import SequenceCache
    ops = _ops(dtype)
    dt = DTYPES[dtype]
    E = H * D
    params = {"width": E, "n_heads": H, "n_kv_heads": K, "head_dim": D, "window": window, "scale": scale,
              "position": {"kind": "rotary", "params": {"head_dim": D, "theta": theta, "pairing": pairing}}}
    part = build_part("mixer", PartSpec("attention", params))
    torch.manual_seed(50)
    # q and k entries of about 1.5: scores spread over a few units, far from uniform attention
    w = {"q": (torch.randn(H * D, E) * 1.5 / math.sqrt(E)).to(dt), "k": (torch.randn(K * D, E) * 1.5 / math.sqrt(E)).to(dt),
         "v": (torch.randn(K * D, E) / math.sqrt(E)).to(dt), "o": (torch.randn(E, H * D) / math.sqrt(E)).to(dt)}
    part.bind({k: v.cuda() for k, v in w.items()}, ops)
    cache = SequenceCache({0: part.cache_need()}, {}, {}, max_tokens=512, max_seq=256, dtype=dt, device=ops.device)
    lens = [70, 13]
    hs = [torch.randn(n, E).to(dt) for n in lens]
    slots = [cache.alloc() for _ in lens]
    outs = [[] for _ in lens]

    def run(chunks):
        for s, _, n in chunks:
            cache.reserve(s, n)
        cache.upload_tables()
        ctx = _ctx(ops, cache, chunks)
        h = torch.cat([hs[slots.index(s)][st:st + n] for s, st, n in chunks]).cuda()
        x = torch.zeros(h.shape[0], E, device="cuda")
        part.forward(ctx, h, 0, accumulate_into=x)
        off = 0
        for s, _, n in chunks:
            outs[slots.index(s)].append(x[off:off + n].cpu())
            off += n
            cache.advance(s, n)

    run([(slots[0], 0, 66), (slots[1], 0, 9)])
    for k in range(4):
        run([(slots[0], 66 + k, 1), (slots[1], 9 + k, 1)])
    cfg = {"num_attention_heads": H, "num_key_value_heads": K, "head_dim": D, "rope_theta": theta,
           "rope_pairing": pairing, "sliding_window": window}
    for i, n in enumerate(lens):
        if scale is None:
            ref, _ = plain.attention_mixer(hs[i].double(), {k: v.double() for k, v in w.items()}, cfg, torch.arange(n))
        else:   # the plain mixer has the default scale; fold the ratio into q
            w2 = {k: v.double() for k, v in w.items()}
            w2["q"] = w2["q"] * (scale * math.sqrt(D))
            ref, _ = plain.attention_mixer(hs[i].double(), w2, cfg, torch.arange(n))
        assert_close(torch.cat(outs[i]), ref, dtype, f"attention part, sequence {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part(dtype):
    """One pre-norm block of tiny A alone on one whole sequence."""
    from rbitnet_b200.config import config_from_dict
    from rbitnet_b200.config.registry import get_architecture
    from rbitnet_b200.parts import build_block
    from rbitnet_b200.cache import SequenceCache
    from rbitnet_b200.weights import random_tensors
    from helpers import sharpen
    ops = _ops(dtype)
    dt = DTYPES[dtype]
    cfg = config_from_dict(TINY_A)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = {k: v.to(dt) for k, v in sharpen(random_tensors(spec, 3), 4.0).items()}
    blk = build_block(spec.layers[1])
    for role, part in blk.parts().items():
        part.bind({k: tensors[spec.layers[1].names[f"{role}.{k}"]].cuda() for k in part.weight_shapes()}, ops)
    cache = SequenceCache({0: blk.mixer.cache_need()}, {}, {}, max_tokens=128, max_seq=128, dtype=dt, device=ops.device)
    s = cache.alloc()
    T = 37
    torch.manual_seed(53)
    cache.reserve(s, T)
    cache.upload_tables()
    x0 = torch.randn(T, cfg.hidden_size)
    x = x0.clone().cuda()
    blk.run(_ctx(ops, cache, [(s, 0, T)]), x, 0)
    ref, _ = plain.block(x0.double(), plain.layer_weights({k: v for k, v in tensors.items()}, 1, torch.float64),
                         plain.normalise_config(TINY_A), torch.arange(T))
    assert_close(x, ref, dtype, "pre-norm block")


# --------------------------------------------------------------------------- the order of layers is data
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_with_a_layer_twice_and_a_shared_cache(tmp_path, dtype):
    """A test architecture made of Llama's parts whose schedule runs layer 0, layer 1, layer 0 again
    (its own cache), then layer 1 reading the keys and values that the FIRST run of layer 1 wrote."""
    from rbitnet_b200 import Engine, StepEntry
    from rbitnet_b200.config import LlamaConfig, register_architecture, unregister_architecture
    from rbitnet_b200.models.llama import build_llama_spec
    from rbitnet_b200.parts import ScheduleEntry

    class LoopedConfig(LlamaConfig):
        architecture: ClassVar[str] = "LoopedTestLM"

    def build(cfg):
        spec = build_llama_spec(cfg)
        spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=1)]
        return spec

    register_architecture("LoopedTestLM", LoopedConfig, build, replace=True)
    try:
        cfgd = dict(TINY_A, architectures=["LoopedTestLM"])
        folder = make_model_dir(tmp_path / "m", cfgd, 4, store=dtype)
        pc, pt = plain.load_folder(folder)
        eng = Engine.load_path(folder, dtype=dtype, max_tokens=1024)
        assert len(eng.cache.groups) == 1 and len(eng.cache.groups[0].entries) == 3     # three caches, one reader
        sched = [(0, None), (1, None), (0, None), (1, 1)]
        ps = prompts([40, 7, 100], cfgd["vocab_size"], 30)
        slots = [eng.new_sequence() for _ in ps]
        lens = [25, 3, 90]
        got = [[] for _ in ps]
        out = eng.step([StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(slots, ps, lens)])
        off = 0
        for i, n in enumerate(lens):
            got[i].append(out[off:off + n])
            off += n
        for k in range(4):
            out = eng.step([StepEntry(s, [p[n + k]], [0]) for s, p, n in zip(slots, ps, lens)])
            for i in range(len(ps)):
                got[i].append(out[i:i + 1])
        for i, (p, n) in enumerate(zip(ps, lens)):
            ref = plain.forward(pc, pt, p[:n + 4], torch.float64, schedule=sched)
            assert_close(torch.cat(got[i]), ref, dtype, f"looped schedule, request {i}")
        plain_default = plain.forward(pc, pt, ps[0][:29], torch.float64)
        assert float((plain_default - plain.forward(pc, pt, ps[0][:29], torch.float64, schedule=sched)).abs().max()) > 1e-3
    finally:
        unregister_architecture("LoopedTestLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,window", [("A", 5), ("B", 64), ("B", 70)])
def test_sliding_window_through_the_engine(tmp_path, dtype, name, window):
    """config.json's sliding_window reaches the kernels: whole prompts, then tokens one by one across
    the window's edge (and across a page's edge for 64 and 70)."""
    from rbitnet_b200 import Engine, StepEntry
    cfgd = dict({"A": TINY_A, "B": TINY_B}[name], sliding_window=window)
    folder = make_model_dir(tmp_path / "m", cfgd, 5, store=dtype)
    ref = PlainModel(folder)
    eng = Engine.load_path(folder, dtype=dtype, max_tokens=1024)
    n = min(cfgd["max_position_embeddings"], 2 * window + 30)
    p = prompts([n], cfgd["vocab_size"], 31)[0]
    full = plain.forward(dict(cfgd, sliding_window=None), ref.tensors, p, torch.float64)
    assert float((full[-1] - ref.logits(p)[-1]).abs().max()) > 1e-4          # the window matters here
    s = eng.new_sequence()
    k = window + 3
    outs = [eng.step([StepEntry(s, p[:k], list(range(k)))])]
    outs += [eng.step([StepEntry(s, [t], [0])]) for t in p[k:]]
    eng.end_sequence(s)
    assert_close(torch.cat(outs), ref.logits(p), dtype, "windowed attention")


# --------------------------------------------------------------------------- a toy mixer with state of its own
def _toy_plain(cfg, tensors, tokens):
    """Plain whole-sequence forward of the toy model below: layer 0 mixes with a decaying running
    sum s_t = decay * s_{t-1} + h_t, y_t = W s_t; layer 1 is ordinary attention."""
    c = plain.normalise_config(cfg)
    t64 = {k: v.double() for k, v in tensors.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = t64["model.embed_tokens.weight"][ids]
    pos = torch.arange(len(tokens))
    h = plain.rmsnorm(x, t64["model.layers.0.input_layernorm.weight"], c["rms_norm_eps"])
    s = torch.zeros(c["hidden_size"], dtype=torch.float64)
    ys = []
    for t in range(len(tokens)):
        s = cfg["decay"] * s + h[t]
        ys.append(t64["model.layers.0.mixer.weight"] @ s)
    x = x + torch.stack(ys)
    lw0 = {k: t64[f"model.layers.0.mlp.{k}_proj.weight"] for k in ("gate", "up", "down")}
    x = x + plain.gated_mlp(plain.rmsnorm(x, t64["model.layers.0.post_attention_layernorm.weight"], c["rms_norm_eps"]), lw0)
    x, _ = plain.block(x, plain.layer_weights(t64, 1, torch.float64), c, pos)
    xn = plain.rmsnorm(x, t64["model.norm.weight"], c["rms_norm_eps"])
    return xn @ t64["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_with_state_can_be_registered_built_and_stepped(tmp_path, dtype):
    from rbitnet_b200 import Engine, StepEntry
    from rbitnet_b200.config import LlamaConfig, register_architecture, unregister_architecture
    from rbitnet_b200.models.llama import build_llama_spec
    from rbitnet_b200.parts import Mixer, StateNeed, PartSpec, register_part, unregister_part
    from rbitnet_b200.weights import random_tensors, write_safetensors

    class DecayMixer(Mixer):
        """y_t = W s_t with s_t = decay * s_{t-1} + h_t kept per sequence in the state area.
        Written with torch on the device: a test part, not a kernel."""

        def __init__(self, width, decay):
            self.width, self.decay = width, decay

        def weight_shapes(self):
            return {"weight": ((self.width, self.width), "matrix")}

        def state_need(self):
            return StateNeed((self.width,), torch.float32)

        def bind(self, weights, ops):
            self.w = weights["weight"].to(torch.float32)

        def forward(self, ctx, h, entry, accumulate_into):
            state = ctx.state_view(entry)                      # [n_slots, width]
            hf = h.to(torch.float32)
            if ctx.meta.single_token:                          # device-only: works inside a captured step
                slots = ctx.meta.tok_slot.long()
                s = self.decay * state[slots] + hf
                state[slots] = s
                accumulate_into += s @ self.w.T
                return
            for c in ctx.meta.seqs:
                s = state[c.slot].clone()
                rows = []
                for t in range(c.n_new):
                    s = self.decay * s + hf[c.offset + t]
                    rows.append(s)
                state[c.slot] = s
                accumulate_into[c.offset:c.offset + c.n_new] += torch.stack(rows) @ self.w.T

    @dataclass
    class ToyConfig(LlamaConfig):
        architecture: ClassVar[str] = "ToyDecayLM"
        decay: float = 0.5

    def build(cfg):
        spec = build_llama_spec(cfg)
        spec.layers[0].mixer = PartSpec("toy_decay", {"width": cfg.hidden_size, "decay": cfg.decay})
        names = {k: v for k, v in spec.layers[0].names.items() if not k.startswith("mixer.")}
        names["mixer.weight"] = "model.layers.0.mixer.weight"
        spec.layers[0].names = names
        return spec

    register_part("mixer", "toy_decay", DecayMixer, replace=True)
    register_architecture("ToyDecayLM", ToyConfig, build, replace=True)
    try:
        cfgd = dict(TINY_B, architectures=["ToyDecayLM"], num_hidden_layers=2, decay=0.8)
        folder = tmp_path / "toy"
        folder.mkdir()
        cfg = ToyConfig.from_dict(cfgd)
        tensors = random_tensors(build(cfg), 6)
        tensors["model.layers.0.mixer.weight"] *= 3
        tensors = {k: v.to(DTYPES[dtype]) for k, v in tensors.items()}
        (folder / "config.json").write_text(json.dumps(cfgd))
        write_safetensors(folder / "model.safetensors", tensors)
        eng = Engine.load_path(folder, dtype=dtype, max_tokens=1024)
        assert list(eng.cache.states) == [0] and eng.cache.states[0].shape[1:] == (cfg.hidden_size,)
        assert len(eng.cache.groups) == 1 and eng.cache.groups[0].entries == [1]      # only layer 1 caches keys
        pc, pt = plain.load_folder(folder)
        for round_ in range(2):                                 # the second round uses the slots again
            ps = prompts([30, 5, 12], cfgd["vocab_size"], 40 + round_)
            lens = [20, 1, 6]
            slots = [eng.new_sequence() for _ in ps]
            got = [[] for _ in ps]
            out = eng.step([StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(slots, ps, lens)])
            off = 0
            for i, n in enumerate(lens):
                got[i].append(out[off:off + n])
                off += n
            for k in range(4):
                out = eng.step([StepEntry(s, [p[n + k]], [0]) for s, p, n in zip(slots, ps, lens)])
                for i in range(len(ps)):
                    got[i].append(out[i:i + 1])
            for i, (p, n) in enumerate(zip(ps, lens)):
                assert_close(torch.cat(got[i]), _toy_plain(pc, pt, p[:n + 4]), dtype, f"toy model round {round_} request {i}")
            for s in slots:
                eng.end_sequence(s)
        # generation (captured decode steps) runs the toy mixer too and keeps its state right
        res = eng.generate([ps[0][:9], ps[2][:4]], max_tokens=5, temperature=0.0)
        for p, r in zip([ps[0][:9], ps[2][:4]], res):
            seq = list(p)
            for t in r.tokens:
                row = _toy_plain(pc, pt, seq)[-1]
                tol = 2 * (TOL[dtype][0] + TOL[dtype][1] * float(row.abs().max()))
                assert float(row[t]) >= float(row.max()) - tol
                seq.append(t)
    finally:
        unregister_architecture("ToyDecayLM")
        unregister_part("mixer", "toy_decay")


# --------------------------------------------------------------------------- a toy feed-forward with routing
def _routed_plain(cfg, tensors, tokens, n_experts):
    """Plain whole-sequence forward of the toy model below: ordinary layers, but the last layer's
    feed-forward sends every token to the one expert (two matrices with a ReLU between) whose router
    logit is largest.  Returns the logits and, per token, how far the two largest router logits are
    apart relative to the largest magnitude (a near tie may go either way under rounding)."""
    c = plain.normalise_config(cfg)
    t64 = {k: v.double() for k, v in tensors.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = t64["model.embed_tokens.weight"][ids]
    pos = torch.arange(len(tokens))
    L = c["num_hidden_layers"]
    for i in range(L - 1):
        x, _ = plain.block(x, plain.layer_weights(t64, i, torch.float64), c, pos)
    lp = f"model.layers.{L - 1}."
    lw = {k: t64[lp + f"self_attn.{k}_proj.weight"] for k in ("q", "k", "v", "o")}
    x = x + plain.attention_mixer(plain.rmsnorm(x, t64[lp + "input_layernorm.weight"], c["rms_norm_eps"]), lw, c, pos)[0]
    h = plain.rmsnorm(x, t64[lp + "post_attention_layernorm.weight"], c["rms_norm_eps"])
    pre = lp + "mlp."
    logits = h @ t64[pre + "router.weight"].T
    top = torch.topk(logits, 2, dim=1).values
    gap = (top[:, 0] - top[:, 1]) / logits.abs().max(dim=1).values
    choice = logits.argmax(dim=1)
    y = torch.zeros_like(x)
    for t in range(len(tokens)):
        e = int(choice[t])
        y[t] = t64[pre + "w2.weight"][e] @ torch.relu(t64[pre + "w1.weight"][e] @ h[t])
    x = x + y
    xn = plain.rmsnorm(x, t64["model.norm.weight"], c["rms_norm_eps"])
    return xn @ t64["lm_head.weight"].T, gap


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_feed_forward_with_routing_can_be_registered_built_and_stepped(tmp_path, dtype):
    """A feed-forward that chooses one of several experts per token (router logits in float32), defined
    here and put into the last layer of an otherwise ordinary model, without a change to the library:
    prompts of unequal lengths, tokens one by one, and captured decode steps through generate()."""
    from rbitnet_b200 import Engine, StepEntry
    from rbitnet_b200.config import LlamaConfig, register_architecture, unregister_architecture
    from rbitnet_b200.models.llama import build_llama_spec
    from rbitnet_b200.parts import FeedForward, PartSpec, register_part, unregister_part
    from rbitnet_b200.weights import random_tensors, write_safetensors
    N_EXPERTS, INNER = 3, 40

    class RoutedExperts(FeedForward):
        """Written with torch on the device, with shapes that do not depend on the routing (every
        expert runs on every row and a mask keeps the chosen one), so that it works inside a
        captured step: a test part, not a kernel."""

        def __init__(self, width, inner, n_experts):
            self.width, self.inner, self.n = width, inner, n_experts

        def weight_shapes(self):
            return {"router": ((self.n, self.width), "matrix"), "w1": ((self.n, self.inner, self.width), "matrix"),
                    "w2": ((self.n, self.width, self.inner), "matrix")}

        def bind(self, weights, ops):
            self.router, self.w1, self.w2 = (weights[k].to(torch.float32) for k in ("router", "w1", "w2"))

        def forward(self, ctx, h, accumulate_into):
            hf = h.to(torch.float32)
            choice = (hf @ self.router.T).argmax(dim=1)                       # float32 logits
            for e in range(self.n):
                y = torch.relu(hf @ self.w1[e].T) @ self.w2[e].T
                accumulate_into += y * (choice == e).to(torch.float32)[:, None]

    @dataclass
    class RoutedConfig(LlamaConfig):
        architecture: ClassVar[str] = "ToyRoutedLM"

    def build(cfg):
        spec = build_llama_spec(cfg)
        last = spec.layers[-1]
        last.feed_forward = PartSpec("toy_routed", {"width": cfg.hidden_size, "inner": INNER, "n_experts": N_EXPERTS})
        names = {k: v for k, v in last.names.items() if not k.startswith("feed_forward.")}
        i = len(spec.layers) - 1
        for k in ("router", "w1", "w2"):
            names[f"feed_forward.{k}"] = f"model.layers.{i}.mlp.{k}.weight"
        last.names = names
        return spec

    register_part("feed_forward", "toy_routed", RoutedExperts, replace=True)
    register_architecture("ToyRoutedLM", RoutedConfig, build, replace=True)
    try:
        cfgd = dict(TINY_B, architectures=["ToyRoutedLM"], num_hidden_layers=2)
        folder = tmp_path / "routed"
        folder.mkdir()
        cfg = RoutedConfig.from_dict(cfgd)
        tensors = random_tensors(build(cfg), 9)
        tensors["model.layers.1.mlp.router.weight"] *= 30          # router logits of order one
        tensors["model.layers.1.mlp.w1.weight"] *= 8
        tensors["model.layers.1.mlp.w2.weight"] *= 8
        tensors = {k: v.to(DTYPES[dtype]) for k, v in tensors.items()}
        (folder / "config.json").write_text(json.dumps(cfgd))
        write_safetensors(folder / "model.safetensors", tensors)
        eng = Engine.load_path(folder, dtype=dtype, max_tokens=1024)
        pc, pt = plain.load_folder(folder)
        min_gap = 1e-4 if dtype == "float32" else 5e-2
        compared = 0
        for round_ in range(2):                                 # the second round uses the slots again
            ps = prompts([30, 5, 12], cfgd["vocab_size"], 50 + round_)
            lens = [20, 1, 6]
            slots = [eng.new_sequence() for _ in ps]
            got = [[] for _ in ps]
            out = eng.step([StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(slots, ps, lens)])
            off = 0
            for i, n in enumerate(lens):
                got[i].append(out[off:off + n])
                off += n
            for k in range(4):
                out = eng.step([StepEntry(s, [p[n + k]], [0]) for s, p, n in zip(slots, ps, lens)])
                for i in range(len(ps)):
                    got[i].append(out[i:i + 1])
            for i, (p, n) in enumerate(zip(ps, lens)):
                want, gap = _routed_plain(pc, pt, p[:n + 4], N_EXPERTS)
                clear = gap > min_gap                            # the routed layer is the last: a near tie touches only its own row
                assert int(clear.sum()) >= (n + 4) * 3 // 4
                assert_close(torch.cat(got[i]).cpu()[clear], want[clear], dtype, f"routed model round {round_} request {i}")
                compared += int(clear.sum())
            for s in slots:
                eng.end_sequence(s)
        assert compared > 60
        probe = torch.randn(64, cfg.hidden_size) @ tensors["model.layers.1.mlp.router.weight"].float().T
        assert len(set(probe.argmax(dim=1).tolist())) == N_EXPERTS        # the router does choose
        # generation (captured decode steps) runs the routed part too
        res = eng.generate([ps[0][:9], ps[2][:4]], max_tokens=5, temperature=0.0)
        assert all(len(r.tokens) == 5 for r in res)
    finally:
        unregister_architecture("ToyRoutedLM")
        unregister_part("feed_forward", "toy_routed")


# --------------------------------------------------------------------------- a toy position encoding
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_position_encoding_can_be_registered_built_and_stepped(tmp_path, dtype, monkeypatch):
    """Another position encoding, defined here: the pairs of a head are rotated with frequencies that
    fall off linearly (1 / (1 + slope * i)) instead of geometrically.  Every attention layer of an
    otherwise ordinary model takes it by name; whole prompts, tokens one by one (where the q/k/v
    product's own epilogue rotates), and generation, against the plain model with the same angles."""
    from rbitnet_b200 import Engine, StepEntry
    from rbitnet_b200.config import LlamaConfig, register_architecture, unregister_architecture
    from rbitnet_b200.models.llama import build_llama_spec
    from rbitnet_b200.parts import PositionEncoding, register_part, unregister_part
    from rbitnet_b200.weights import random_tensors, write_safetensors

    def frequencies(head_dim, slope):
        return 1.0 / (1.0 + slope * torch.arange(head_dim // 2, dtype=torch.float32))

    class LinearFrequencies(PositionEncoding):
        def __init__(self, head_dim, slope, pairing):
            self.head_dim, self.slope, self.pairing = head_dim, slope, pairing

        def bind(self, weights, ops):
            self.inv_freq = frequencies(self.head_dim, self.slope).to(ops.device)

        def rotary(self):
            return self.inv_freq, self.pairing == "interleaved", self.head_dim

    @dataclass
    class ToyConfig(LlamaConfig):
        architecture: ClassVar[str] = "ToyLinearRopeLM"
        slope: float = 0.5

    def build(cfg):
        spec = build_llama_spec(cfg)
        for layer in spec.layers:
            layer.mixer.params["position"] = {"kind": "toy_linear_frequencies",
                                              "params": {"head_dim": cfg.head_dim, "slope": cfg.slope,
                                                         "pairing": cfg.rope_pairing}}
        return spec

    register_part("position", "toy_linear_frequencies", LinearFrequencies, replace=True)
    register_architecture("ToyLinearRopeLM", ToyConfig, build, replace=True)
    try:
        cfgd = dict(TINY_A, architectures=["ToyLinearRopeLM"], slope=0.25)
        folder = tmp_path / "toyrope"
        folder.mkdir()
        cfg = ToyConfig.from_dict(cfgd)
        tensors = {k: v.to(DTYPES[dtype]) for k, v in sharpen(random_tensors(build(cfg), 4), 4.0).items()}
        (folder / "config.json").write_text(json.dumps(cfgd))
        write_safetensors(folder / "model.safetensors", tensors)
        eng = Engine.load_path(folder, dtype=dtype, max_tokens=1024)
        pc, pt = plain.load_folder(folder)
        inv = frequencies(cfg.head_dim, cfg.slope)
        monkeypatch.setattr(plain, "rope_angles", lambda positions, head_dim, theta: positions.to(torch.float32)[:, None] * inv[None, :])
        ps = prompts([40, 3, 17], cfgd["vocab_size"], 61)
        lens = [33, 1, 9]
        slots = [eng.new_sequence() for _ in ps]
        got = [[] for _ in ps]
        out = eng.step([StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(slots, ps, lens)])
        off = 0
        for i, n in enumerate(lens):
            got[i].append(out[off:off + n])
            off += n
        for k in range(2):
            out = eng.step([StepEntry(s, [p[n + k]], [0]) for s, p, n in zip(slots, ps, lens)])
            for i in range(len(ps)):
                got[i].append(out[i:i + 1])
        for i, (p, n) in enumerate(zip(ps, lens)):
            assert_close(torch.cat(got[i]), plain.forward(pc, pt, p[:n + 2]), dtype, f"toy rope request {i}")
        # and the encoding matters: the ordinary geometric frequencies give other logits
        monkeypatch.undo()
        other = plain.forward(pc, pt, ps[0][:lens[0] + 2])
        assert float((torch.cat(got[0]).double().cpu() - other).abs().max()) > 1e-2 * float(other.abs().max())
        for s in slots:
            eng.end_sequence(s)
        res = eng.generate([ps[0][:9], ps[2][:4]], max_tokens=4, temperature=0.0)
        assert all(len(r.tokens) == 4 for r in res)
    finally:
        unregister_architecture("ToyLinearRopeLM")
        unregister_part("position", "toy_linear_frequencies")


@pytest.mark.parametrize("head_dim,theta", [(16, 10000.0), (48, 500000.0), (128, 1e6)])
def test_position_encoding_part(head_dim, theta):
    """The rotary part's inverse frequencies are the reference's 1/theta^(2i/D) in float32
    (crates/bitnet-core/src/llama/model.rs:126-127); 'none' gives no rotation."""
    from rbitnet_b200.parts import build_part, PartSpec
    ops = _ops("float32")
    for pairing in ("half", "interleaved"):
        part = build_part("position", PartSpec("rotary", {"head_dim": head_dim, "theta": theta, "pairing": pairing}))
        part.bind({}, ops)
        inv, interleaved, rot = part.rotary()
        assert interleaved == (pairing == "interleaved") and rot == head_dim
        pos = torch.tensor([1000])
        want = plain.rope_angles(pos, head_dim, theta)[0] / 1000.0
        assert torch.allclose(inv.cpu(), want, rtol=1e-6, atol=0)
    assert build_part("position", PartSpec("none", {})).rotary() is None
    with pytest.raises(ValueError, match="even"):
        build_part("position", PartSpec("rotary", {"head_dim": 15, "theta": 1e4}))


def test_decode_with_more_than_16_heads_per_kv_head_through_captured_steps(tmp_path):
    """Multi-query attention with 20 query heads on one kv head: the decode step takes the prefill
    kernels (the split decode kernel holds at most 16 heads per group), also when captured."""
    from rbitnet_b200 import Engine
    cfg = dict(TINY_B, num_attention_heads=20, num_key_value_heads=1, head_dim=64, hidden_size=1280,
               intermediate_size=520, num_hidden_layers=1)
    folder = make_model_dir(tmp_path / "m", cfg, 8, store="bfloat16", factor=1.0)
    ref = PlainModel(folder)
    eng = Engine.load_path(folder, dtype="bfloat16", max_tokens=1024)
    ps = prompts([70, 3], cfg["vocab_size"], 70)
    res = eng.generate(ps, max_tokens=4, temperature=0.0)
    for p, r in zip(ps, res):
        full = ref.logits(list(p) + r.tokens)
        for i, t in enumerate(r.tokens):
            row = full[len(p) - 1 + i]
            assert float(row[t]) >= float(row.max()) - 4e-2 * float(row.abs().max())


# --------------------------------------------------------------------------- other blocks, other cache contents, scales
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_block_of_three_norms_a_one_vector_cache_a_rotated_prefix_and_scales(tmp_path, dtype):
    """A toy architecture, defined and registered here, that needs of the framework what Llama does not:
    layer 0 is another arrangement of parts with a third norm (after the mixer, before the residual sum)
    and a mixer that keeps ONE vector per position in the cache (no keys and values) and returns the mean
    of all of them so far; layer 1 is an ordinary block whose attention rotates only the first half of
    every head; the embedding is multiplied by 2 and the logits by 0.5.  Whole prompts, tokens one by one,
    captured decode steps and slots used again, against plain formulas written out below."""
    from rbitnet_b200 import Engine, StepEntry
    from rbitnet_b200.config import LlamaConfig, register_architecture, unregister_architecture
    from rbitnet_b200.models.llama import build_llama_spec
    from rbitnet_b200.parts import (Mixer, CacheNeed, PartSpec, PositionEncoding, register_part, unregister_part,
                                    build_part)
    from rbitnet_b200.parts.block import build_parts
    from rbitnet_b200.weights import random_tensors, write_safetensors
    KEEP = 40          # width of the vector the toy mixer keeps per position

    class MeanMixer(Mixer):
        def __init__(self, width, keep):
            self.width, self.keep = width, keep

        def weight_shapes(self):
            return {"keep": ((self.keep, self.width), "matrix"), "out": ((self.width, self.keep), "matrix")}

        def cache_need(self):
            return CacheNeed(1, self.keep, streams=((1, self.keep),))

        def bind(self, weights, ops):
            self.w_keep, self.w_out = weights["keep"].to(torch.float32), weights["out"].to(torch.float32)

        def forward(self, ctx, h, entry, accumulate_into):
            view, meta = ctx.cache_view(entry), ctx.meta
            assert view.v is None and len(view.streams) == 1
            store = view.streams[0]                                   # [pages, 1, page, keep]
            slot, pos = meta.tok_slot.long(), meta.tok_pos.long()
            c = h.to(torch.float32) @ self.w_keep.T
            page = view.page_table.long()[slot, pos // view.page_size]
            store[page, 0, pos % view.page_size] = c.to(store.dtype)
            # every row reads its sequence's pages in full and masks by position: shapes do not depend
            # on the data, so the same code runs inside a captured step
            pages = view.page_table.long()[slot]                      # [T, max_pages]
            kept = store[pages, 0].to(torch.float32).reshape(len(slot), -1, self.keep)
            seen = (torch.arange(kept.shape[1], device=kept.device)[None, :] <= pos[:, None]).to(torch.float32)
            mean = (kept * seen[:, :, None]).sum(1) / (pos + 1).to(torch.float32)[:, None]
            accumulate_into += mean @ self.w_out.T

    class SandwichBlock:
        def __init__(self, spec):
            self._parts = build_parts(spec)

        def parts(self):
            return self._parts

        def run(self, ctx, x, entry):
            p = self._parts
            y = torch.zeros_like(x)
            p["mixer"].forward(ctx, p["mixer_norm"].forward(ctx, x), entry, accumulate_into=y)
            x += p["post_norm"].forward(ctx, y).to(torch.float32)
            p["feed_forward"].forward(ctx, p["ffn_norm"].forward(ctx, x), accumulate_into=x)

    class PrefixRotary(PositionEncoding):
        def __init__(self, rot_dim, theta, pairing):
            self.rot_dim, self.theta, self.pairing = rot_dim, theta, pairing

        def bind(self, weights, ops):
            i = torch.arange(self.rot_dim // 2, dtype=torch.float32)
            self.inv_freq = (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), 2.0 * i / self.rot_dim)).to(ops.device)

        def rotary(self):
            return self.inv_freq, self.pairing == "interleaved", self.rot_dim

    @dataclass
    class ToyConfig(LlamaConfig):
        architecture: ClassVar[str] = "ToySandwichLM"

    def build(cfg):
        spec = build_llama_spec(cfg)
        first = spec.layers[0]
        first.arrangement = "toy_sandwich"
        first.mixer = PartSpec("toy_mean", {"width": cfg.hidden_size, "keep": KEEP})
        first.post_norm = PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps}, role="norm")
        names = {k: v for k, v in first.names.items() if not k.startswith("mixer.")}
        names.update({"mixer.keep": "model.layers.0.mixer.keep.weight", "mixer.out": "model.layers.0.mixer.out.weight",
                      "post_norm.weight": "model.layers.0.post_mixer_layernorm.weight"})
        first.names = names
        spec.layers[1].mixer.params["position"] = {"kind": "toy_prefix_rotary", "params": {
            "rot_dim": cfg.head_dim // 2, "theta": cfg.rope_theta, "pairing": cfg.rope_pairing}}
        spec.embedding_scale, spec.logit_scale = 2.0, 0.5
        return spec

    def toy_plain(cfg, tensors, tokens):
        c = plain.normalise_config(cfg)
        t = {k: v.double() for k, v in tensors.items()}
        ids = torch.as_tensor(tokens, dtype=torch.long)
        pos = torch.arange(len(tokens))
        eps = c["rms_norm_eps"]
        x = t["model.embed_tokens.weight"][ids] * 2.0
        p0 = "model.layers.0."
        lw = {"gate": t[p0 + "mlp.gate_proj.weight"], "up": t[p0 + "mlp.up_proj.weight"], "down": t[p0 + "mlp.down_proj.weight"],
              "attn_norm": t[p0 + "input_layernorm.weight"], "ffn_norm": t[p0 + "post_attention_layernorm.weight"]}
        kept = plain.rmsnorm(x, lw["attn_norm"], eps) @ t["model.layers.0.mixer.keep.weight"].T
        mean = torch.cumsum(kept, 0) / (pos + 1).double()[:, None]
        x = x + plain.rmsnorm(mean @ t["model.layers.0.mixer.out.weight"].T, t["model.layers.0.post_mixer_layernorm.weight"], eps)
        x = x + plain.gated_mlp(plain.rmsnorm(x, lw["ffn_norm"], eps), lw)
        lw = plain.layer_weights(t, 1, torch.float64)
        H, K, D = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        h = plain.rmsnorm(x, lw["attn_norm"], eps)
        q, k = (h @ lw["q"].T).reshape(-1, H, D), (h @ lw["k"].T).reshape(-1, K, D)
        v = (h @ lw["v"].T).reshape(-1, K, D)
        R = D // 2
        q = torch.cat([plain.rope(q[..., :R], pos, c["rope_theta"], c["rope_pairing"]), q[..., R:]], dim=-1)
        k = torch.cat([plain.rope(k[..., :R], pos, c["rope_theta"], c["rope_pairing"]), k[..., R:]], dim=-1)
        x = x + plain.attention(q, k, v) @ lw["o"].T
        x = x + plain.gated_mlp(plain.rmsnorm(x, lw["ffn_norm"], eps), lw)
        return plain.rmsnorm(x, t["model.norm.weight"], eps) @ t["lm_head.weight"].T * 0.5

    register_part("mixer", "toy_mean", MeanMixer, replace=True)
    register_part("block", "toy_sandwich", SandwichBlock, replace=True)
    register_part("position", "toy_prefix_rotary", PrefixRotary, replace=True)
    register_architecture("ToySandwichLM", ToyConfig, build, replace=True)
    try:
        cfgd = dict(TINY_B, architectures=["ToySandwichLM"], num_hidden_layers=2)
        cfg = ToyConfig.from_dict(cfgd)
        spec = build(cfg)
        table = spec.tensor_table()
        assert table["model.layers.0.post_mixer_layernorm.weight"] == ((cfg.hidden_size,), "norm")
        assert "model.layers.0.self_attn.q_proj.weight" not in table and "model.layers.1.self_attn.q_proj.weight" in table
        tensors = {k: v.to(DTYPES[dtype]) for k, v in sharpen(random_tensors(spec, 12), 4.0).items()}
        folder = tmp_path / "sandwich"
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(cfgd))
        write_safetensors(folder / "model.safetensors", tensors)
        eng = Engine.load_path(folder, dtype=dtype, max_tokens=1024)
        shapes = sorted(tuple(p.shape[2:]) for g in eng.cache.groups for p in g.pools)
        assert shapes == sorted([(1, 64, KEEP), (1, 64, cfg.head_dim), (1, 64, cfg.head_dim)])   # one vector; keys and values
        pc, pt = plain.load_folder(folder)
        for round_ in range(2):
            ps = prompts([100, 9, 70], cfgd["vocab_size"], 90 + round_)
            lens = [62, 3, 64]
            slots = [eng.new_sequence() for _ in ps]
            got = [[] for _ in ps]
            out = eng.step([StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(slots, ps, lens)])
            off = 0
            for i, n in enumerate(lens):
                got[i].append(out[off:off + n])
                off += n
            for k in range(6):
                out = eng.step([StepEntry(s, [p[n + k]], [0]) for s, p, n in zip(slots, ps, lens)], captured=k % 2 == 1)
                for i in range(len(ps)):
                    got[i].append(out[i:i + 1])
            for i, (p, n) in enumerate(zip(ps, lens)):
                assert_close(torch.cat(got[i]), toy_plain(pc, pt, p[:n + 6]), dtype, f"sandwich round {round_} request {i}")
            for s in slots:
                eng.end_sequence(s)
        # the scales and the rotated prefix matter: the ordinary model on the same weights gives other logits
        res = eng.generate([ps[0][:9], ps[2][:4]], max_tokens=4, temperature=0.0)
        assert all(len(r.tokens) == 4 for r in res)
    finally:
        unregister_architecture("ToySandwichLM")
        for role, kind in (("mixer", "toy_mean"), ("block", "toy_sandwich"), ("position", "toy_prefix_rotary")):
            unregister_part(role, kind)
