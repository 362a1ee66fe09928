"""Decode throughput of the Llama-3-8B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

A step is one decode step: one token for each of ``batch`` sequences whose cache already
holds ``prompt_len`` tokens.  ``value`` is decoded tokens a second with the step chained on
the device (the sampled ids feed the next step there); ``e2e`` is the same step driven
through the engine's Python entry point with host token ids in and sampled ids out every
step.  The line also carries a 2,048-token prefill, the decode step's memory roofline, and
decode at batch 1 and 64.  Weights are random (there is no checkpoint to load) and the
cache content is random; the work does not depend on either.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: the Llama-3-8B shape
MODEL = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
             num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
             rms_norm_eps=1e-5, max_position_embeddings=8192, tie_word_embeddings=False, hidden_act="silu")
FULL_LAYERS = 32
PROMPT_LEN = 2048
METRIC = "decode tok/s @ batch 8 (Llama-3-8B shape, 2048-token prompts, bf16)"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self, t0, t1):
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 7] or [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


def fill_cache(engine, batch, context, room):
    """``batch`` live sequences of ``context`` cached positions each (random keys and values),
    with pages reserved for ``room`` more."""
    import torch
    slots = []
    for _ in range(batch):
        s = engine.new_sequence()
        engine.cache.reserve(s, context + room)
        engine.cache.advance(s, context)
        slots.append(s)
    engine.cache.upload_tables()
    return slots


def decode_bytes(engine, batch, context):
    """What a decode step has to read: every weight it uses once, and the live sequences' cache."""
    w = engine.model.weight_bytes()      # every matrix a step multiplies by (the embedding table is only gathered from)
    per_token = sum(g.bytes_per_position()
                    for g in engine.cache.groups)
    return w + batch * context * per_token


def time_decode(engine, batch, context, steps, warmup, sampler=None):
    """Device-chained decode steps, timed with CUDA events.  Returns (ms per step, launches per step,
    clock summary)."""
    import torch
    slots = fill_cache(engine, batch, context, steps + warmup + 8)
    g = engine.decode_graph(batch)
    g.stage(slots, [1] * batch, [context] * batch, [0.0] * batch, [0.5] * batch)
    if g.graph is None:
        g.capture(pool=engine._graph_pool)
        if engine._graph_pool is None:
            engine._graph_pool = g.graph.pool()
    g.stage(slots, [1] * batch, [context] * batch, [0.0] * batch, [0.5] * batch)
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = engine.ops.lib.launches
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    launches = engine.ops.lib.launches - before
    ms = e0.elapsed_time(e1) / steps
    engine.ops.check_errors()
    for s in slots:
        engine.end_sequence(s)
    clocks = sampler.summary(t0, t1) if sampler else None
    return ms, launches, clocks


def time_decode_e2e(engine, batch, context, steps, warmup):
    """The same step through Engine: host token ids in (pinned copy), sampled ids out, every step."""
    import torch
    slots = fill_cache(engine, batch, context, 0)
    feed = [(s, [1]) for s in slots]
    temps, us = [0.0] * batch, [0.5] * batch
    for _ in range(warmup):
        ids = engine._step_sample(feed, temps, us)
        feed = [(s, [i]) for s, i in zip(slots, ids)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        ids = engine._step_sample(feed, temps, us)
        feed = [(s, [i]) for s, i in zip(slots, ids)]
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    g = engine.decode_graph(batch)
    for s in slots:
        engine.end_sequence(s)
    return dt / steps * 1e3, g.h2d_bytes, g.d2h_bytes


def time_generate(engine, batch, context, steps, warmup):
    """Decode through ``Engine.generate`` itself: ``batch`` prompts of ``context`` host token ids in, every
    generated id out through ``on_token``; the time between the first token after ``warmup + 64`` steps
    and the last one, by the host's clock.  The 64 further steps are left out because the steps of the
    first 0.1 s after a prompt of this size run up to 18 % slower, at the clocks the power limit left
    after the prefill (the same captured step, replayed after a second's pause, is as fast as on a cache
    that no prefill filled).  generate launches a decode step before it has read the ids of the step
    before, so this is not the plain step of ``e2e``; it is reported beside it."""
    import torch
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, engine.config.vocab_size, (context,), generator=g).tolist() for _ in range(batch)]
    stamps = []

    def on_token(request, token):
        if request == 0:
            stamps.append(time.perf_counter())

    skip = warmup + 64
    engine.generate(prompts, max_tokens=skip + steps + 1, temperature=0.0, stop_ids=[], on_token=on_token)
    torch.cuda.synchronize()
    if len(stamps) < skip + steps + 1:
        return None
    return (stamps[skip + steps] - stamps[skip]) / steps * 1e3


def time_prefill(engine, tokens, reps=3):
    import torch
    from rbitnet_b200 import StepEntry
    ids = torch.randint(0, engine.config.vocab_size, (tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    times = []
    for r in range(reps + 1):
        s = engine.new_sequence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        out = engine.step([StepEntry(s, ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        assert bool(torch.isfinite(out).all())
        engine.end_sequence(s)
        if r > 0:
            times.append(e0.elapsed_time(e1))
    return min(times)


def prefill_flops(cfg, layers, tokens):
    E, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, K, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = 2 * tokens * (E * (H + 2 * K) * D + H * D * E + 3 * E * F)
    attn = 4 * H * D * tokens * (tokens + 1) / 2
    return layers * (per_layer + attn) + 2 * E * V


# The other generation workloads of BASELINE.json (configs[3] and configs[4]), run through Engine.generate.
WORKLOADS = {
    "llama2_7b_unequal": dict(
        model=dict(architectures=["LlamaForCausalLM"], num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                   num_key_value_heads=32, head_dim=128, intermediate_size=11008, vocab_size=32000, rope_theta=10000.0,
                   rms_norm_eps=1e-5, max_position_embeddings=4096),
        prompts=16, len_lo=64, len_hi=2048, max_tokens=256, temperature=0.0),
    "tinyllama_b64_sampling": dict(
        model=dict(architectures=["LlamaForCausalLM"], num_hidden_layers=22, hidden_size=2048, num_attention_heads=32,
                   num_key_value_heads=4, head_dim=64, intermediate_size=5632, vocab_size=32000, rope_theta=10000.0,
                   rms_norm_eps=1e-5, max_position_embeddings=2048),
        prompts=64, len_lo=512, len_hi=512, max_tokens=1024, temperature=0.8),
}


def run_workload(name):
    """End-to-end generation (host token ids in, generated ids out) of one of WORKLOADS; one short line."""
    import torch
    from rbitnet_b200 import Engine
    w = WORKLOADS[name]
    cfg = w["model"]
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(w["len_lo"], w["len_hi"] + 1, (w["prompts"],), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    cache_tokens = sum(-(-(n + w["max_tokens"]) // 64) * 64 for n in lens) + 4096
    eng = Engine.from_random(cfg, seed=1, dtype="bfloat16", max_tokens=cache_tokens,
                             max_seq=cfg["max_position_embeddings"], max_batch=64)
    times = []
    for _ in range(2):                     # the first run also captures the decode steps
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = eng.generate(prompts, max_tokens=w["max_tokens"], temperature=w["temperature"], seed=3, stop_ids=[])
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    new = sum(len(r.tokens) for r in res)
    print(json.dumps({"workload": name, "layers": cfg["num_hidden_layers"], "prompts": len(prompts),
                      "prompt_tokens": sum(lens), "new_tokens": new, "seconds": round(times[1], 3),
                      "first_run_seconds": round(times[0], 3), "new_tokens_per_s": round(new / times[1], 1),
                      "steps": eng.last_stats["steps"], "temperature": w["temperature"], "dtype": "bf16",
                      "data": "synthetic (random weights and token ids)"}))
    return 0


def print_timeline(engine, batch, context):
    """When each kernel of one captured decode step really ran (CUPTI records through torch.profiler,
    no replay, no serialisation): with programmatic dependent launch a kernel starts early and
    waits, so the useful figure per kernel is how long after the previous kernel's end it ended."""
    import torch
    from torch.profiler import profile, ProfilerActivity
    slots = fill_cache(engine, batch, context, 64)
    g = engine.decode_graph(batch)
    g.stage(slots, [1] * batch, [context] * batch, [0.0] * batch, [0.5] * batch)
    if g.graph is None:
        g.capture(pool=engine._graph_pool)
    g.stage(slots, [1] * batch, [context] * batch, [0.0] * batch, [0.5] * batch)
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                key=lambda e: e.time_range.start)
    last = ev[-(len(ev) // 3):]
    t0, prev_end = last[0].time_range.start, last[0].time_range.start
    print(f"{'start':>9} {'end':>9} {'after prev end':>15}  kernel   (microseconds from the step's first kernel)")
    for e in last:
        end = e.time_range.end
        print(f"{e.time_range.start - t0:9.1f} {end - t0:9.1f} {end - max(prev_end, t0):15.1f}  {e.name[:80]}")
        prev_end = max(prev_end, end)
    print(f"step: {prev_end - t0:.1f} us, {len(last)} kernels")
    for s_ in slots:
        engine.end_sequence(s_)


class KernelTimer:
    """Times every operation of a step with CUDA events around its launch(es), by wrapping the methods
    of the engine's kernel layer.  The step must run kernel by kernel (not as a captured graph).  An
    event between two launches ends the overlap that programmatic dependent launch gives neighbours,
    so these are the times of the kernels alone, each starting on an idle GPU: their sum is above the
    step's own time, and a kernel's share of its roofline here is a lower bound of what it reaches
    inside the step."""
    decode_context = 0     # cached positions per sequence of the decode step being described without a sync
    OPS = ("embed", "rmsnorm", "linear", "gated_linear", "project_rotate_append", "rotate_append", "attention",
           "gather_rows", "sample", "decode_advance")

    def __init__(self, ops, events=True):
        """events=False: only note, per operation, what it is and how many kernels it launched."""
        self.ops, self.records, self._depth, self._saved, self.events = ops, [], 0, {}, events

    def __enter__(self):
        import torch
        for name in self.OPS:
            fn = getattr(self.ops, name)
            self._saved[name] = fn

            def wrapped(*a, _fn=fn, _name=name, **kw):
                if self._depth:                        # an operation made of others is timed as a whole
                    return _fn(*a, **kw)
                self._depth += 1
                e0 = e1 = None
                before = self.ops.lib.launches
                if self.events:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                try:
                    out = _fn(*a, **kw)
                finally:
                    self._depth -= 1
                if self.events:
                    e1.record()
                    self.records.append((_name, self._describe(_name, a, kw), e0, e1))
                else:
                    self.records.append((_name, self._describe(_name, a, kw, sync=False), self.ops.lib.launches - before, None))
                return out
            setattr(self.ops, name, wrapped)
        return self

    def __exit__(self, *exc):
        for name, fn in self._saved.items():
            setattr(self.ops, name, fn)

    @staticmethod
    def _describe(name, a, kw, sync=True):
        """(label, bytes the operation has to move, flops).  sync=False: nothing is read back from the
        device (inside a capture); a decode's keys are then counted from the step's longest context."""
        el = lambda t: t.numel() * t.element_size()
        if name in ("linear", "gated_linear", "project_rotate_append"):
            x, w = a[0], a[1]
            pending = hasattr(x, "squares")       # rows with their norm pending: the bfloat16 rows and the sums of squares
            extra = el(x.squares) if pending else 0
            x = x.scaled if pending else x
            T, K = x.shape
            N = w.w.shape[0]
            n_out = getattr(w, "inner", N)
            out_b = T * n_out * (4 if (kw.get("out_dtype") is not None and kw["out_dtype"].itemsize == 4) else 2)
            if kw.get("accumulate_into") is not None:
                out_b = 2 * T * n_out * 4
            kind = {"linear": "product", "gated_linear": "gate/up product + SiLU*up",
                    "project_rotate_append": "q/k/v product + rotation + append"}[name]
            if kw.get("accumulate_into") is not None:
                kind = "product + residual"
            if pending:
                kind = "norm's factor, " + kind
            if kw.get("then_norm") is not None and T <= 16:
                kind += " + next norm's rows"
                extra += T * n_out * 2
            return f"{kind} [{T}x{K}]x[{N}x{K}]", el(w.w) + el(x) + out_b + extra, 2.0 * T * N * K
        if name == "attention":
            q, meta, view, H = a[0], a[1], a[2], a[3]
            T, _, D = q.shape
            if not meta.single_token:
                keys = sum(c.start + c.n_new for c in meta.seqs)
                seen = sum(c.n_new * c.start + c.n_new * (c.n_new + 1) // 2 for c in meta.seqs)
            elif sync:
                keys = seen = int(meta.tok_pos.sum()) + T
            else:
                keys = seen = T * KernelTimer.decode_context
            flops = 4.0 * H * D * seen
            return (f"attention {'decode' if meta.single_token else 'prefill'} [{T} tokens, {H}/{view.n_kv_heads} heads of {D}]",
                    keys * view.n_kv_heads * D * 2 * q.element_size() + 2 * el(q), flops)
        if name in ("rmsnorm", "embed", "gather_rows", "rotate_append"):
            t = a[0]
            return f"{name} [{t.shape[0]} rows]", 2 * el(t) if name != "embed" else t.shape[0] * a[1].shape[1] * 6, 0.0
        if name == "sample":
            return f"sample [{a[0].shape[0]} rows of {a[0].shape[1]}]", el(a[0]), 0.0
        return name, 0, 0.0

    def table(self, pk, reps, times_us=None):
        """Aggregated over equal labels: [{label, calls per step, us per call, GB/s, TFLOP/s, frac}].
        ``times_us``: the operations' times if they were not taken with events."""
        import torch
        torch.cuda.synchronize()
        agg = {}
        for i, (name, (label, nbytes, flops), e0, e1) in enumerate(self.records):
            d = agg.setdefault(label, {"calls": 0, "us": 0.0, "bytes": nbytes, "flops": flops})
            d["calls"] += 1
            d["us"] += times_us[i] if times_us is not None else e0.elapsed_time(e1) * 1e3
        rows = []
        for label, d in agg.items():
            us = d["us"] / d["calls"]
            bound_us = max(d["bytes"] / (pk["hbm_gbs"] * 1e9), d["flops"] / (pk["bf16_tflops"] * 1e12)) * 1e6
            rows.append({"kernel": label, "calls_per_step": round(d["calls"] / reps, 2), "us": round(us, 2),
                         "gb_s": round(d["bytes"] / us / 1e3, 1), "tflop_s": round(d["flops"] / us / 1e6, 2),
                         "bound": "hbm" if d["bytes"] / (pk["hbm_gbs"] * 1e9) >= d["flops"] / (pk["bf16_tflops"] * 1e12) else "tensor",
                         "frac": round(bound_us / us, 3) if us > 0 else None,
                         "share_of_step": None})
        total = sum(r["us"] * r["calls_per_step"] for r in rows)
        for r in rows:
            r["share_of_step"] = round(r["us"] * r["calls_per_step"] / total, 3)
        rows.sort(key=lambda r: -r["share_of_step"])
        return rows, total


def kernel_tables(engine, batch, ctx, prefill_tokens, pk, reps=5):
    """Per-kernel times, rates and roofline fractions of one decode step and one prefill step
    (roofline = max(bytes / copy bandwidth, flops / burst tensor rate), both measured).  The decode
    step's kernels take microseconds, less than a pair of events costs, so they are timed inside the
    captured step from CUPTI's records; the prefill step's kernels are timed with CUDA events around
    each operation (its inputs are on the device before the timed run, and the GPU idles for some
    milliseconds first, so that the host has queued the whole step by the time its first kernel
    starts and no event interval holds a wait for the host)."""
    import numpy as np
    import torch
    from rbitnet_b200.engine.step import SeqChunk, StepContext, build_meta
    out = {}
    # ---- decode: the captured step as it runs.  The operations are noted (what, how many kernels) while
    # the step is captured; CUPTI's records of one replay then give, per kernel, how long after the end
    # of the kernel before it it ended: that is what it adds to the step, overlap included.
    from torch.profiler import profile, ProfilerActivity
    slots = fill_cache(engine, batch, ctx, 64)
    engine._graphs.pop(batch, None)
    g = engine.decode_graph(batch)
    g.stage(slots, [1] * batch, [ctx] * batch, [0.0] * batch, [0.5] * batch)
    KernelTimer.decode_context = ctx
    g._body()                                           # the trial run, so that the capture below is the only noted run
    torch.cuda.synchronize()
    g.stage(slots, [1] * batch, [ctx] * batch, [0.0] * batch, [0.5] * batch)
    with KernelTimer(engine.ops, events=False) as kt:
        noted = []
        g.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g.graph, pool=engine._graph_pool):
            g.sampled = g._body()
        noted = list(kt.records)
        g.stage(slots, [1] * batch, [ctx] * batch, [0.0] * batch, [0.5] * batch)
        for _ in range(5):
            g.graph.replay()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                g.graph.replay()
            torch.cuda.synchronize()
        ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
        n_kernels = sum(r[2] for r in noted)
        last = ev[-n_kernels:] if len(ev) >= 3 * n_kernels else []
        times, prev_end, i = [], (last[0].time_range.start if last else 0.0), 0
        for _, _, n, _ in noted:
            t = 0.0
            for e in last[i:i + n]:
                t += max(0.0, e.time_range.end - prev_end)
                prev_end = max(prev_end, e.time_range.end)
            i += n
            times.append(t)
        kt.records = noted
        rows, total = kt.table(pk, 1, times_us=times) if last else ([], 0.0)
    engine._graphs.pop(batch, None)                     # captured by hand here: not for the engine to use
    out["decode"] = {"batch": batch, "context": ctx, "step_us": round(total, 1), "kernels_per_step": n_kernels,
                     "how": "captured step, time each kernel adds after the one before it ended", "kernels": rows}
    for s in slots:
        engine.end_sequence(s)
    ids = torch.randint(0, engine.config.vocab_size, (prefill_tokens,), generator=torch.Generator().manual_seed(1))
    s = engine.new_sequence()
    engine.cache.reserve(s, prefill_tokens)
    engine.cache.upload_tables()
    meta = build_meta([SeqChunk(s, 0, prefill_tokens, 0)], ids.numpy().astype(np.int32),
                      np.asarray([prefill_tokens - 1], dtype=np.int32), engine.ops.device)
    ctx_ = StepContext(engine.ops, meta, engine.cache)
    engine.model.forward(ctx_)                           # also makes the attention's tile lists
    torch.cuda.synchronize()
    with KernelTimer(engine.ops) as kt:
        torch.cuda._sleep(40_000_000)
        engine.model.forward(ctx_)
        rows, total = kt.table(pk, 1)
    engine.end_sequence(s)
    out["prefill"] = {"tokens": prefill_tokens, "sum_of_kernels_us": round(total, 1),
                      "how": "kernel by kernel, CUDA events around each operation", "kernels": rows}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip prefill and the batch 1/64 points")
    ap.add_argument("--phase", default="all", choices=["all", "prefill"],
                    help="'prefill': only the 2,048-token prefill, one short line (for profiling)")
    ap.add_argument("--context", type=int, default=PROMPT_LEN,
                    help="cached positions per sequence when the decode steps begin (default: the 2,048 of the headline; "
                         "other values are for further measurements and are named in config.seq_len)")
    ap.add_argument("--prefill-tokens", type=int, default=PROMPT_LEN,
                    help="with --phase prefill: the prompt's length (up to 8,000), for profiling other lengths")
    ap.add_argument("--kernels", action="store_true",
                    help="time every kernel of one decode step and one prefill step alone (CUDA events around eager "
                         "launches) and print, per kernel, time, GB/s, TFLOP/s and the fraction of its roofline")
    ap.add_argument("--timeline", action="store_true",
                    help="print when each kernel of one decode step ran inside the captured graph, and exit")
    ap.add_argument("--shape", default="llama3_8b", choices=["llama3_8b", "llama2_7b", "tinyllama_1b"],
                    help="layer sizes of the decode and prefill measurements (default: the headline's; the others "
                         "are those of the generation workloads and are named in metric and config)")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="run one of the other generation workloads end to end instead (one short line)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "azerothl/Rbitnet is a Rust workspace: no Rust toolchain in this image, no network to get "
                          "one, and it loads GGUF files only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload:
        return run_workload(args.workload)
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    import torch
    from rbitnet_b200 import Engine
    pk = peaks()
    shape_name, model = {"llama3_8b": ("Llama-3-8B shape", MODEL),
                         "llama2_7b": ("Llama-2-7B shape", WORKLOADS["llama2_7b_unequal"]["model"]),
                         "tinyllama_1b": ("TinyLlama-1.1B shape", WORKLOADS["tinyllama_b64_sampling"]["model"])}[args.shape]
    full_layers, max_seq = model["num_hidden_layers"], model["max_position_embeddings"]
    layers = full_layers if args.layers == FULL_LAYERS else min(args.layers, full_layers)
    cfg = dict(model, num_hidden_layers=layers)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    room = steps + warmup + 64 + 16     # time_generate leaves 64 further steps out
    ctx = max(1, min(max_seq - room, args.context))
    max_tokens = max(b * (-(-(max(ctx, PROMPT_LEN) + room) // 64) * 64) for b in batches) + 64 * 64
    t_build = time.time()
    engine = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_seq=max_seq, max_batch=64)
    for g in engine.cache.groups:                   # random cache content; finite values, no work depends on it
        for pool in g.pools:
            pool.normal_(0.0, 1.0)
    torch.cuda.synchronize()
    build_s = time.time() - t_build

    if args.timeline:
        print_timeline(engine, args.batch, ctx)
        return 0
    if args.kernels:
        tables = kernel_tables(engine, args.batch, ctx, min(PROMPT_LEN, args.prefill_tokens), pk)
        print(json.dumps({"kernels_of": shape_name, "layers": layers, "peaks": pk, **tables}))
        for phase in ("decode", "prefill"):
            t = tables[phase]
            print(f"\n{phase} ({t['how']}): {t.get('step_us', t.get('sum_of_kernels_us')):.1f} us", file=sys.stderr)
            print(f"{'us':>9} {'calls':>6} {'share':>6} {'GB/s':>8} {'TFLOP/s':>8} {'bound':>6} {'frac':>6}  kernel", file=sys.stderr)
            for r in t["kernels"]:
                print(f"{r['us']:9.1f} {r['calls_per_step']:6.1f} {r['share_of_step']:6.3f} {r['gb_s']:8.1f} "
                      f"{r['tflop_s']:8.2f} {r['bound']:>6} {r['frac']:6.3f}  {r['kernel']}", file=sys.stderr)
        return 0
    if args.phase == "prefill":
        n_tok = max(1, min(8000, args.prefill_tokens))
        pf_ms = time_prefill(engine, n_tok, reps=max(1, min(3, steps)))
        print(json.dumps({"phase": "prefill", "tokens": n_tok, "layers": layers, "ms": round(pf_ms, 3),
                          "tokens_per_s": round(n_tok / pf_ms * 1e3, 1)}))
        return 0

    sampler = ClockSampler().start()
    try:
        ms, launches, clocks = time_decode(engine, args.batch, ctx, steps, warmup, sampler)
        e2e_ms, h2d, d2h = time_decode_e2e(engine, args.batch, ctx, steps, warmup)
        gen_ms = None if args.no_points else time_generate(engine, args.batch, ctx, steps, warmup)
        points, prefill = {}, None
        if not args.no_points:
            for b in (1, 64):
                if b == args.batch:
                    points[f"decode_b{b}"] = round(b / ms * 1e3, 1)
                else:
                    pms, _, _ = time_decode(engine, b, ctx, steps, warmup)
                    points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
            pf_ms = time_prefill(engine, PROMPT_LEN)
            flops = prefill_flops(cfg, layers, PROMPT_LEN)
            prefill = {"value": round(PROMPT_LEN / pf_ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(pf_ms, 3),
                       "frac": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                       "peak_tflops": pk["bf16_tflops_sustained"], "peak": f"bf16 sustained, {pk['source']}",
                       "frac_burst": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                       "peak_tflops_burst": pk["bf16_tflops"]}
    finally:
        sampler.stop()

    nbytes = decode_bytes(engine, args.batch, ctx)
    metric = METRIC.replace("Llama-3-8B shape", shape_name).replace("batch 8", f"batch {args.batch}")
    if ctx != PROMPT_LEN:
        metric = metric.replace("2048-token", f"{ctx}-token")
    achieved = nbytes / (ms * 1e-3) / 1e9
    value = args.batch / ms * 1e3
    line = {
        "metric": metric, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, random token ids, random cache)",
        "impl": "ours",
        "config": {"model": shape_name, "layers": layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"], "tied_head": False,
                   "global_batch": args.batch, "seq_len": ctx, "max_context": max_seq,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read once per step)",
                   "step": "one decode token per sequence, CUDA graph, sampled on device"},
        "e2e": {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes,
                     "peak_source": pk["source"]},
        "build_s": round(build_s, 1),
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
    if gen_ms:
        line["generate"] = {"value": round(args.batch / gen_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(gen_ms, 4),
                            "what": "the same decode steps through Engine.generate (host prompts in, ids out by "
                                    "callback; a step is launched ahead of the ids it reads)"}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
