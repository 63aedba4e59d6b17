#!/usr/bin/env python3
"""Decode and prefill throughput of the library on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--config gptj6b|codegen2b|codegen16b] [--skip-points] [--per-kernel]

The default run has GPT-J-6B's layer sizes (28 layers, width 4096, 16 heads of 256, rotary 64,
inner 16384, vocabulary 50400, 2048 positions) with random bfloat16 weights, a batch of 8
sequences and a context of 2048: a "step" is one decode step (one token for each of the 8
sequences) whose last timed step fills the context.  `value` is decoded tokens per second
on the device (CUDA events around exactly K steps); `e2e` is the same K steps through the
Python entry point `qstream_b200.generate` with host token lists in and out (timed on the host
between the arrival of the tokens of step W' and of the last step); `prefill` times one
2,048-token prompt; `roofline` compares the decode step's bytes (every weight once, the cache
of the live sequences) with the measured copy bandwidth.

`points` holds decode at batch 1 and 64 at context 2048, and, for batch 1, 8 and 64, a whole
run from 128-token prompts until the context is full (1,920 steps): tokens per second
averaged over the run and at contexts 128, 1088 and 2048, each with its fraction of the copy
bandwidth; and the wall-clock time of a step with short prompts (1 x 128 and 8 x 64 tokens), replayed from
a captured graph and, for comparison, launched kernel by kernel.  `codegen2b` and `codegen16b` are the two other benchmark shapes of the GPT-J
architecture (16 prompts of unequal lengths with 256 decoded tokens each; a 2,048-token
prefill and decode at batch 32 from 512-token prompts).  `--config` runs one shape alone;
`--per-kernel` times each kernel of one layer by itself (CUDA events around a captured graph
of many repeats, each repeat on another layer's weights so that nothing is served from L2) and prints a table of
achieved GB/s or TFLOP/s against the measured peaks.  `--batch B --context C --skip-points` times decode steps
at another point; a context beyond the shape's 2,048 positions lengthens the position table and nothing else.

Inputs are synthetic token ids, uniform over the vocabulary; each step reads more than
5 GB, far more than the 126 MB L2, so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = {
    "gptj6b": dict(n_layer=28, n_embd=4096, n_head=16, n_positions=2048, vocab_size=50400, rotary_dim=64,
                   n_inner=16384, activation_function="gelu_new", layer_norm_epsilon=1e-5,
                   architectures=["GPTJForCausalLM"]),
    "codegen2b": dict(n_layer=32, n_embd=2560, n_head=32, n_positions=2048, vocab_size=51200, rotary_dim=64,
                      n_inner=10240, activation_function="gelu_new", layer_norm_epsilon=1e-5,
                      architectures=["GPTJForCausalLM"]),
    "codegen16b": dict(n_layer=34, n_embd=6144, n_head=24, n_positions=2048, vocab_size=51200, rotary_dim=64,
                       n_inner=24576, activation_function="gelu_new", layer_norm_epsilon=1e-5,
                       architectures=["GPTJForCausalLM"]),
}
NAMES = {"gptj6b": "GPT-J-6B sizes", "codegen2b": "CodeGen-2B sizes (GPT-J architecture)",
         "codegen16b": "CodeGen-16B sizes (GPT-J architecture)"}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as fh:
            d = json.load(fh)
        for k in FALLBACK_PEAKS:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index=0):
        self.lines, self.proc, self.thread = [], None, None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(index), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        return time.time()

    def summary(self, t0, t1):
        rows = [l for t, l in self.lines if t0 <= t <= t1 + 0.25] or [l for _, l in self.lines[-3:]]
        sm, mx, reasons = [], 0, set()
        for line in rows:
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(int(float(parts[0])))
                mx = max(mx, int(float(parts[1])))
            except (ValueError, IndexError):
                continue
            for name, v in zip(self.NAMES, parts[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()


def reference_arm():
    # QStream is a CPU-only C program without a Python package (no setup.py or pyproject.toml), so
    # a `pip install` of its source tree has nothing to install; its converter cannot read a GPT-J
    # folder and its engine has no GPT-J forward pass or unquantized weights.
    print(json.dumps({"impl": "reference",
                      "unavailable": "QStream is a CPU-only C engine with no Python package to install; its "
                                     "converter rejects GPT-J folders and its engine does not compute GPT-J"}))
    return 0


class Bench:
    """One model shape on the device, with the measurements that the JSON line is made of."""

    def __init__(self, shape: str, n_layer: int, sampler: ClockSampler, pk: dict, seed: int = 0, n_positions: int = 0):
        import numpy as np
        import torch
        import qstream_b200 as qs
        self.np, self.torch, self.qs = np, torch, qs
        self.shape, self.pk, self.sampler = shape, pk, sampler
        self.n_layer_full = SHAPES[shape]["n_layer"]
        sizes = {**SHAPES[shape], "n_layer": n_layer or self.n_layer_full}
        if n_positions > sizes["n_positions"]:            # a context beyond the shape's own: the same layers, a longer position table
            sizes["n_positions"] = n_positions
        self.cfg = qs.GptjConfig.from_dict(sizes)
        self.model = qs.CausalLM.random(self.cfg, seed=seed, dtype="bfloat16", device="cuda:0")
        self.rng = np.random.default_rng(seed)
        c = self.cfg
        self.kv_bytes_per_token = 2 * c.n_layer * c.n_embd * 2
        self.weight_bytes = self.model.weight_bytes - self.model.embedding_bytes    # every weight a step reads

    def close(self):
        self.model = None
        self.torch.cuda.empty_cache()

    def prompts(self, lengths):
        return [[int(t) for t in self.rng.integers(0, self.cfg.vocab_size, n)] for n in lengths]

    def step_bytes(self, batch, mean_ctx):
        return self.weight_bytes + batch * self.cfg.n_embd * 2 + batch * mean_ctx * self.kv_bytes_per_token

    def hbm_frac(self, batch, mean_ctx, ms):
        return self.step_bytes(batch, mean_ctx) / (ms * 1e-3) / 1e9 / self.pk["hbm_gbs"]

    # ------------------------------------------------------------------ decode on the device
    def _decoder(self, engine, slots, logits):
        """A function that runs one decode step as the generation loop does: the sampled tokens feed the
        next step on the device, and the host reads every step's tokens (a copy into pinned memory) while
        the following step runs."""
        torch, qs = self.torch, self.qs
        from qstream_b200.csrc import ops
        from qstream_b200.engine import TokenFeed
        batch = len(slots)
        state = {"tokens": ops.argmax(logits), "turn": 0}
        host = [torch.empty(batch, dtype=torch.int32).pin_memory() for _ in range(2)]
        copied = [None, None]
        rows = list(range(batch))

        def one_step():
            out = engine.step(slots, TokenFeed(state["tokens"], rows))
            state["tokens"] = ops.argmax(out)
            turn = state["turn"]
            host[turn].copy_(state["tokens"], non_blocking=True)
            copied[turn] = torch.cuda.Event()
            copied[turn].record()
            state["turn"] = turn ^ 1
            if copied[turn ^ 1] is not None:
                copied[turn ^ 1].synchronize()
                host[turn ^ 1].tolist()
        return one_step

    def _prefill_all(self, engine, slots, prompts, chunk_tokens=4096):
        torch = self.torch
        per = max(1, chunk_tokens // max(len(p) for p in prompts))
        logits = []
        for a in range(0, len(slots), per):
            logits.append(engine.step(slots[a:a + per], prompts[a:a + per]).clone())
        return torch.cat(logits)

    def decode_at_context(self, batch, ctx, steps, warmup):
        """Prefill `batch` prompts so that the last timed decode step fills the context; time `steps`
        decode steps (greedy sampling on the device included) with CUDA events."""
        torch, qs = self.torch, self.qs
        from qstream_b200.csrc import ops
        engine = qs.Engine(self.model, max_tokens=batch * ctx, max_batch=batch, max_context=ctx)
        slots = [engine.acquire() for _ in range(batch)]
        one_step = self._decoder(engine, slots, self._prefill_all(engine, slots, self.prompts([ctx - (steps + warmup)] * batch)))
        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = self.sampler.mark()
        start.record()
        for _ in range(steps):
            one_step()
        stop.record()
        torch.cuda.synchronize()
        t1 = self.sampler.mark()
        ms = start.elapsed_time(stop) / steps
        engine.check_status()
        launches = ops.launch_count() - launches0
        mean_ctx = ctx - steps / 2.0
        for s in slots:
            engine.release(s)
        del engine
        torch.cuda.empty_cache()
        return {"tok_s": batch * 1000.0 / ms, "ms": ms, "launches": launches, "bytes": self.step_bytes(batch, mean_ctx),
                "frac": self.hbm_frac(batch, mean_ctx, ms), "clocks": self.sampler.summary(t0, t1)}

    def decode_run(self, batch, prompt_len, ctx, window=32, marks=()):
        """A whole run: `batch` prompts of `prompt_len` tokens, then one token each until the context is
        full.  An event every `window` steps gives the step time along the run; `marks` are contexts at
        which tokens per second are reported (the window that starts there, or the last one)."""
        torch, qs = self.torch, self.qs
        engine = qs.Engine(self.model, max_tokens=batch * ctx, max_batch=batch, max_context=ctx)
        engine.capture_decode_graphs([batch])                      # every graph the run will replay, before the clock starts
        warm = [engine.acquire() for _ in range(batch)]
        step = self._decoder(engine, warm, self._prefill_all(engine, warm, self.prompts([8] * batch)))
        for _ in range(4):
            step()
        for s in warm:
            engine.release(s)
        slots = [engine.acquire() for _ in range(batch)]
        one_step = self._decoder(engine, slots, self._prefill_all(engine, slots, self.prompts([prompt_len] * batch)))
        n_steps = ctx - prompt_len
        torch.cuda.synchronize()
        events = [torch.cuda.Event(enable_timing=True)]
        events[0].record()
        for i in range(n_steps):
            one_step()
            if (i + 1) % window == 0 or i + 1 == n_steps:
                events.append(torch.cuda.Event(enable_timing=True))
                events[-1].record()
        torch.cuda.synchronize()
        engine.check_status()
        total_ms = events[0].elapsed_time(events[-1])
        out = {"avg": batch * n_steps * 1000.0 / total_ms,
               "avg_frac": self.hbm_frac(batch, (prompt_len + ctx) / 2.0, total_ms / n_steps)}
        n_windows = len(events) - 1
        for c in marks:
            w = min(max(0, (c - prompt_len) // window), n_windows - 1)
            first, last = w * window, min((w + 1) * window, n_steps)
            ms = events[w].elapsed_time(events[w + 1]) / (last - first)
            mean_ctx = prompt_len + (first + last) / 2.0
            out[f"c{c}"] = batch * 1000.0 / ms
            out[f"c{c}_frac"] = self.hbm_frac(batch, mean_ctx, ms)
        for s in slots:
            engine.release(s)
        del engine
        torch.cuda.empty_cache()
        return out

    # ------------------------------------------------------------------ prefill
    def prefill_flops(self, lengths):
        c = self.cfg
        D, F, H, dh, V = c.n_embd, c.inner, c.n_head, c.head_dim, c.vocab_size
        T = sum(lengths)
        attn = sum(2 * 2 * dh * H * n * (n + 1) / 2 for n in lengths)
        return c.n_layer * (2 * T * D * (3 * D) + 2 * T * D * D + 2 * 2 * T * D * F + attn) + len(lengths) * 2 * D * V

    def prefill(self, lengths, repeats=5):
        """One step with prompts of the given lengths; time to the logits of their last positions."""
        torch, qs = self.torch, self.qs
        T = sum(lengths)
        engine = qs.Engine(self.model, max_tokens=sum(-(-n // 64) * 64 for n in lengths), max_batch=len(lengths),
                           max_context=max(lengths))
        prompts = self.prompts(lengths)
        times = []
        for _ in range(repeats):
            slots = [engine.acquire() for _ in lengths]
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            engine.step(slots, prompts)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            for s in slots:
                engine.release(s)
        engine.check_status()
        ms = sorted(times[2:])[len(times[2:]) // 2]
        del engine
        torch.cuda.empty_cache()
        return {"value": round(T * 1000.0 / ms, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(self.prefill_flops(lengths) / (ms * 1e-3) / (self.pk["bf16_tflops"] * 1e12), 4)}

    def short_prompts(self, n_seq, length, use_graphs=True, repeats=9):
        """Wall-clock milliseconds of one step with `n_seq` prompts of `length` tokens (host lists in, logits on
        the device, the device awaited): what a caller waits for.  Steps of this size are bound by the host when
        launched kernel by kernel; `use_graphs` replays them as one captured graph."""
        torch, qs = self.torch, self.qs
        engine = qs.Engine(self.model, max_tokens=n_seq * (-(-length // 64) * 64), max_batch=n_seq,
                           max_context=length, use_graphs=use_graphs)
        prompts = self.prompts([length] * n_seq)
        times = []
        for _ in range(repeats):
            slots = [engine.acquire() for _ in range(n_seq)]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.step(slots, prompts)
            torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) * 1e3)
            for s in slots:
                engine.release(s)
        engine.check_status()
        del engine
        torch.cuda.empty_cache()
        return sorted(times[2:])[len(times[2:]) // 2]

    # ------------------------------------------------------------------ through the Python entry point
    def end_to_end(self, batch, ctx, steps, settle=48):
        """`qstream_b200.generate` with host token lists in and out.  The timed region is the last `steps`
        decode steps, between the moments at which the host holds the tokens of step `settle` and of the
        last step: every step copies its metadata from pinned host memory and reads the chosen tokens
        back.  The steps before let the clocks settle after the prefill."""
        qs = self.qs
        from qstream_b200.engine.graphs import bucket_for
        engine = qs.Engine(self.model, max_tokens=batch * ctx, max_batch=batch, max_context=ctx)
        engine.capture_decode_graphs([batch])
        greedy = qs.SamplingConfig.greedy()
        qs.generate(engine, self.prompts([64] * batch), max_new_tokens=4, sampling=greedy, stop_tokens=())
        total = settle + steps
        prompts = self.prompts([ctx - total] * batch)
        stamps = []

        def callback(i, tok):
            if i == 0:
                stamps.append(time.perf_counter())
        t0 = self.sampler.mark()
        res = qs.generate(engine, prompts, max_new_tokens=total + 1, sampling=greedy, stop_tokens=(), callback=callback)
        t1 = self.sampler.mark()
        assert all(len(t) == total + 1 for t in res.tokens) and len(stamps) == total + 1
        seconds = stamps[-1] - stamps[settle]
        del engine
        self.torch.cuda.empty_cache()
        return {"value": round(batch * steps / seconds, 2), "unit": "tokens/s",
                "h2d_bytes_per_step": (8 * bucket_for(batch) + 1) * 4, "d2h_bytes_per_step": batch * 4,
                "whole_call_tok_s": round(res.decode_tokens / res.decode_seconds, 2),
                "prefill_tok_s": round(res.prefill_tokens / res.prefill_seconds, 1),
                "clocks": self.sampler.summary(t0, t1)}

    def unequal_batch(self, lengths, new_tokens):
        """Prompts of unequal lengths in one prefill step, then `new_tokens` tokens each through the entry
        point; decode tokens per second over the whole call and the bandwidth fraction at the mean context."""
        qs = self.qs
        batch = len(lengths)
        ctx = max(lengths) + new_tokens
        engine = qs.Engine(self.model, max_tokens=sum(-(-(n + new_tokens) // 64) * 64 for n in lengths), max_batch=batch,
                           max_context=ctx)
        greedy = qs.SamplingConfig.greedy()
        engine.capture_decode_graphs([batch])
        qs.generate(engine, self.prompts([16] * batch), max_new_tokens=4, sampling=greedy, stop_tokens=())
        res = qs.generate(engine, self.prompts(lengths), max_new_tokens=new_tokens, sampling=greedy, stop_tokens=())
        assert all(len(t) == new_tokens for t in res.tokens)
        ms = res.decode_seconds * 1000.0 / (new_tokens - 1)
        mean_ctx = sum(lengths) / batch + new_tokens / 2.0
        del engine
        self.torch.cuda.empty_cache()
        return {"decode_tok_s": round(res.decode_tokens / res.decode_seconds, 1), "ms_per_step": round(ms, 3),
                "hbm_frac": round(self.hbm_frac(batch, mean_ctx, ms), 4),
                "prefill_tok_s": round(res.prefill_tokens / res.prefill_seconds, 1), "prefill_tokens": res.prefill_tokens}


def run_codegen2b(sampler, pk, layers=0):
    import numpy as np
    b = Bench("codegen2b", layers, sampler, pk, seed=2)
    lengths = [int(n) for n in np.random.default_rng(2).integers(32, 1025, 16)]
    out = {"n_layer": b.cfg.n_layer, "n_layer_full": b.n_layer_full, "batch": 16, "prompt_tokens": sum(lengths),
           "new_tokens": 256}
    out.update(b.unequal_batch(lengths, 256))
    pf = b.prefill(lengths)
    out["prefill_device_tok_s"], out["prefill_frac"] = pf["value"], pf["frac"]
    b.close()
    return out


def run_codegen16b(sampler, pk, layers=0):
    b = Bench("codegen16b", layers, sampler, pk, seed=4)
    out = {"n_layer": b.cfg.n_layer, "n_layer_full": b.n_layer_full}
    pf = b.prefill([2048])
    out["prefill_tok_s"], out["prefill_ms"], out["prefill_frac"] = pf["value"], pf["ms"], pf["frac"]
    r = b.decode_run(32, 512, 512 + 256, window=64, marks=(512,))
    out.update({"decode_batch": 32, "decode_from": 512, "decode_steps": 256, "decode_tok_s": round(r["avg"], 1),
                "decode_hbm_frac": round(r["avg_frac"], 4)})
    b.close()
    return out


# ----------------------------------------------------------------------------- each kernel alone

def per_kernel(shape, layers, pk, batch, ctx, prefill_tokens=2048, repeats=56):
    """Each kernel of one layer by itself, as the step calls it: CUDA events around `repeats` launches, each
    repeat on another layer's weights and cache entry so that nothing is served from L2."""
    import torch
    import qstream_b200 as qs
    from qstream_b200.csrc import attention_bf16, ops
    from qstream_b200.engine.step import StepContext
    from qstream_b200.parts.linear import linear

    n_layer = max(layers or 8, 4)
    sizes = {**SHAPES[shape], "n_layer": n_layer}
    sizes["n_positions"] = max(sizes["n_positions"], ctx, prefill_tokens + 1)      # longer contexts: a longer position table
    cfg = qs.GptjConfig.from_dict(sizes)
    model = qs.CausalLM.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    D, F, H, dh, V = cfg.n_embd, cfg.inner, cfg.n_head, cfg.head_dim, cfg.vocab_size
    rng = torch.Generator(device="cuda").manual_seed(0)
    rows = []

    def timed(name, fn, bytes_=0, flops=0):
        # the repeats are captured into one CUDA graph, as a decode step is: the host's launch cost is not timed
        for i in range(3):
            fn(i % n_layer)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(repeats):
                fn(i % n_layer)
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1000.0 / repeats
        gbs = bytes_ / us / 1e3
        tfl = flops / us / 1e6
        rows.append({"kernel": name, "us": round(us, 2), "GB/s": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 3),
                     "TFLOP/s": round(tfl, 1), "tc_frac": round(tfl / pk["bf16_tflops"], 3)})

    for phase, T, lengths in (("decode", batch, [ctx - 1] * batch), ("prefill", prefill_tokens, [prefill_tokens])):
        engine = qs.Engine(model, max_tokens=sum(-(-(n + 1) // 64) * 64 for n in lengths), max_batch=len(lengths),
                           max_context=max(lengths) + 1, use_graphs=False)
        slots = [engine.acquire() for _ in lengths]
        if phase == "decode":               # fill the cache, then build the metadata of one decode step
            engine.cache.prepare(slots, [n for n in lengths])
            engine.cache.commit(slots, [n for n in lengths])
            for g in engine.cache.groups:
                g.k.normal_(generator=rng)
                g.v.normal_(generator=rng)
            sb = engine.build_batch(slots, [[1]] * len(slots))
        else:
            sb = engine.build_batch(slots, [[1] * n for n in lengths])
        step = StepContext(sb, engine.cache, engine.status, None)
        x = torch.randn(T, D, device="cuda", generator=rng).bfloat16()
        blocks = model.blocks
        h = blocks[0].norms["input"].forward(x)
        hidden = torch.empty(T, D + F, dtype=torch.bfloat16, device="cuda")
        qkv = linear(h, blocks[0].mixer.w_qkv)
        kv_read = sum(min(n, ctx) for n in lengths) * 2 * D * 2 if phase == "decode" else 0
        causal = sum(2 * 2 * dh * H * n * (n + 1) / 2 for n in lengths)
        tag = f"{phase} T={T}"
        timed(f"{tag} layernorm", lambda i: blocks[i].norms["input"].forward(x), bytes_=2 * T * D * 2)
        timed(f"{tag} q/k/v product", lambda i: linear(h, blocks[i].mixer.w_qkv), bytes_=3 * D * D * 2, flops=2 * T * D * 3 * D)

        def rope(i):
            m = blocks[i].mixer
            view = step.kv(i)
            ops.rope_store(qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:], H, H, dh, m.position.rotary_dim, m.position.fused_table,
                           sb.tok_slot, sb.tok_pos, view.page_table, view.page_tokens, view.k, view.v, step.status, settled=True)
        timed(f"{tag} rotary + cache write", rope, bytes_=T * 3 * D * 2 + T * 2 * D * 2)

        def attend(i):
            m = blocks[i].mixer
            attention_bf16.attend(qkv[:, :D], m.spec, step, step.kv(i), hidden[:, :D])
        timed(f"{tag} attention", attend, bytes_=kv_read, flops=causal if phase == "prefill" else 0)
        timed(f"{tag} fc_in product + gelu", lambda i: blocks[i].ffn.forward_hidden(h, step, out=hidden[:, D:]),
              bytes_=D * F * 2, flops=2 * T * D * F)
        timed(f"{tag} out_proj + fc_out product + residual",
              lambda i: linear(hidden, blocks[i].fused_weight, blocks[i].fused_bias, residuals=(x,)),
              bytes_=(D + F) * D * 2, flops=2 * T * (D + F) * D)
        if phase == "decode":
            # the same two projections as the block runs them when the feed-forward goes beside the mixer
            mm = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
            timed(f"{tag} fc_out product alone", lambda i: linear(hidden[:, D:], blocks[i].fused_weight[:, D:], blocks[i].fused_bias, out=mm),
                  bytes_=F * D * 2, flops=2 * T * F * D)
            timed(f"{tag} out_proj product + residuals", lambda i: linear(hidden[:, :D], blocks[i].fused_weight[:, :D], None, residuals=(x, mm)),
                  bytes_=D * D * 2, flops=2 * T * D * D)
            z = torch.randn(T, D, device="cuda", generator=rng).bfloat16()
            logits = model.head.forward(z)
            timed(f"{tag} lm_head product", lambda i: model.head.forward(z),
                  bytes_=V * D * 2, flops=2 * T * D * V)
            timed(f"{tag} argmax", lambda i: ops.argmax(logits), bytes_=T * V * 4)
        engine.check_status()
        del engine, step, sb
        torch.cuda.empty_cache()
    print(f"# {NAMES[shape]}, one layer's kernels, batch {batch}, context {ctx}; peaks {pk['source']}: "
          f"{pk['hbm_gbs']} GB/s, {pk['bf16_tflops']} TFLOP/s; the lm_head product and argmax repeat on one matrix "
          f"(larger than L2)")
    print(f"{'kernel':58s} {'us':>9s} {'GB/s':>9s} {'of copy':>8s} {'TFLOP/s':>9s} {'of bf16':>8s}")
    for r in rows:
        print(f"{r['kernel']:58s} {r['us']:9.2f} {r['GB/s']:9.1f} {r['hbm_frac']:8.3f} {r['TFLOP/s']:9.1f} {r['tc_frac']:8.3f}")
    print(json.dumps({"per_kernel": rows}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="gptj6b", choices=sorted(SHAPES), help="which benchmark shape (default: gptj6b)")
    ap.add_argument("--skip-points", action="store_true", help="the timed steps only: no other batch sizes, runs, prefill, e2e")
    ap.add_argument("--per-kernel", action="store_true", help="time each kernel of one layer by itself and print a table")
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="with --per-kernel: tokens of the prompt step")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    torch.cuda.set_device(0)
    pk = peaks()
    if args.per_kernel:
        return per_kernel(args.config, args.layers, pk, args.batch, args.context, args.prefill_tokens)
    sampler = ClockSampler(0)
    if args.config != "gptj6b":
        fn = run_codegen2b if args.config == "codegen2b" else run_codegen16b
        out = fn(sampler, pk, args.layers)
        sampler.stop()
        print(json.dumps({"impl": "ours", "config": {"model": NAMES[args.config]}, "dtype": "bf16",
                          "data": "synthetic token ids, random weights", args.config: out}))
        return 0

    bench = Bench("gptj6b", args.layers, sampler, pk, n_positions=args.context)
    cfg, ctx = bench.cfg, args.context
    main_run = bench.decode_at_context(args.batch, ctx, args.steps, args.warmup)
    gbs = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": "GPT-J-6B bf16 decode tok/s @ batch 8, context 2048",
        "value": round(main_run["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
        "impl": "ours",
        "config": {"model": NAMES["gptj6b"], "n_layer": cfg.n_layer, "n_layer_full": bench.n_layer_full,
                   "n_embd": cfg.n_embd, "n_head": cfg.n_head, "head_dim": cfg.head_dim,
                   "rotary_dim": cfg.rotary, "n_inner": cfg.inner, "vocab_size": cfg.vocab_size,
                   "n_positions": cfg.n_positions, "global_batch": args.batch, "seq_len": ctx,
                   "parallelism": "single GPU", "sampling": "greedy on device",
                   "l2": "inputs larger than L2 (step reads >12 GB)", "peaks": pk["source"]},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4)},
    }

    if not args.skip_points:
        points = {}
        for b, name in ((1, "decode_b1"), (64, "decode_b64")):
            r = bench.decode_at_context(b, ctx, min(args.steps, 32), max(3, min(args.warmup, 4)))
            points[name] = round(r["tok_s"], 2)
            points[name + "_hbm_frac"] = round(r["frac"], 4)
        line["prefill"] = bench.prefill([2048])
        line["e2e"] = bench.end_to_end(args.batch, ctx, args.steps)
        # whole runs from 128-token prompts until the context is full
        for b in (1, 8, 64):
            r = bench.decode_run(b, 128, ctx, window=32, marks=(128, 1088, 2048))
            points[f"run_b{b}_avg"] = round(r["avg"], 1)
            points[f"run_b{b}_avg_hbm_frac"] = round(r["avg_frac"], 4)
            for c in (128, 1088, 2048):
                points[f"run_b{b}_c{c}"] = round(r[f"c{c}"], 1)
                points[f"run_b{b}_c{c}_hbm_frac"] = round(r[f"c{c}_frac"], 4)
        # steps with short prompts: wall-clock, replayed from a captured graph and launched kernel by kernel
        for n_seq, length in ((1, 128), (8, 64)):
            points[f"prefill_{n_seq}x{length}_ms"] = round(bench.short_prompts(n_seq, length), 3)
            points[f"prefill_{n_seq}x{length}_eager_ms"] = round(bench.short_prompts(n_seq, length, use_graphs=False), 3)
        line["points"] = points
        bench.close()
        del bench
        for name, fn in (("codegen2b", run_codegen2b), ("codegen16b", run_codegen16b)):
            try:                                    # the headline line is printed whatever happens to the extra shapes
                line[name] = fn(sampler, pk)
            except Exception as e:                  # noqa: BLE001
                line[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()
    sampler.stop()
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
