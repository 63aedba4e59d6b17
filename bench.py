#!/usr/bin/env python3
"""Decode and prefill throughput of the library on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

The default run has GPT-J-6B's layer sizes (28 layers, width 4096, 16 heads of 256, rotary 64,
inner 16384, vocabulary 50400, 2048 positions) with random bfloat16 weights, a batch of 8
sequences and a context of 2048: a "step" is one decode step (one token for each of the 8
sequences) whose last timed step fills the context.  `value` is decoded tokens per second
on the device (CUDA events around exactly K steps); `e2e` is the same through the Python
entry point `qstream_b200.generate` with host token lists in and out; `prefill` times one
2,048-token prompt; `points` holds decode at batch 1 and 64; `roofline` compares the decode
step's bytes (every weight once, the cache of the live sequences) with the measured copy
bandwidth.  Inputs are synthetic token ids, uniform over the vocabulary; each step reads more
than 12 GB, far more than the 126 MB L2, so no L2 flush is needed between steps.
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

GPTJ_6B = dict(n_layer=28, n_embd=4096, n_head=16, n_positions=2048, vocab_size=50400, rotary_dim=64,
               n_inner=16384, activation_function="gelu_new", layer_norm_epsilon=1e-5,
               architectures=["GPTJForCausalLM"])
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the 28 of the configuration (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64, prefill and e2e")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch
    import qstream_b200 as qs
    from qstream_b200.csrc import ops

    torch.cuda.set_device(0)
    pk = peaks()
    n_layer = args.layers or GPTJ_6B["n_layer"]
    cfg = qs.GptjConfig.from_dict({**GPTJ_6B, "n_layer": n_layer})
    model = qs.CausalLM.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(0)
    V, ctx = cfg.vocab_size, args.context
    sampler = ClockSampler(0)

    kv_bytes_per_token = 2 * n_layer * cfg.n_embd * 2

    def decode_run(batch, steps, warmup):
        """Prefill `batch` prompts so that the last timed decode step fills the context; time `steps`
        decode steps (greedy sampling on the device included) with CUDA events."""
        engine = qs.Engine(model, max_tokens=batch * ctx, max_batch=batch, max_context=ctx)
        prompt_len = ctx - (steps + warmup)
        slots = [engine.acquire() for _ in range(batch)]
        prompts = [[int(t) for t in rng.integers(0, V, prompt_len)] for _ in range(batch)]
        chunk = max(1, 4096 // prompt_len)
        logits = []
        for a in range(0, batch, chunk):
            logits.append(engine.step(slots[a:a + chunk], prompts[a:a + chunk]))
        tokens = ops.argmax(torch.cat(logits))       # stays on the device
        host = [torch.empty(batch, dtype=torch.int32).pin_memory() for _ in range(2)]
        copied = [None, None]
        turn = 0

        def one_step():
            # As the generation loop does it: the sampled tokens feed the next step on the device, and the
            # host reads every step's tokens (a copy into pinned memory) while the following step runs.
            nonlocal tokens, turn
            out = engine.step(slots, tokens)
            tokens = ops.argmax(out)
            host[turn].copy_(tokens, non_blocking=True)
            copied[turn] = torch.cuda.Event()
            copied[turn].record()
            turn ^= 1
            if copied[turn] is not None:
                copied[turn].synchronize()
                host[turn].tolist()

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = sampler.mark()
        start.record()
        for _ in range(steps):
            one_step()
        stop.record()
        torch.cuda.synchronize()
        t1 = sampler.mark()
        ms = start.elapsed_time(stop) / steps
        engine.check_status()
        launches = ops.launch_count() - launches0
        mean_ctx = ctx - steps / 2.0
        step_bytes = model.weight_bytes - model.wte.numel() * 2 + batch * cfg.n_embd * 2 \
            + batch * mean_ctx * kv_bytes_per_token
        for s in slots:
            engine.release(s)
        del engine
        torch.cuda.empty_cache()
        return {"tok_s": batch * 1000.0 / ms, "ms": ms, "launches": launches, "bytes": step_bytes,
                "clocks": sampler.summary(t0, t1)}

    main_run = decode_run(args.batch, args.steps, args.warmup)
    gbs = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": "GPT-J-6B bf16 decode tok/s @ batch 8, context 2048",
        "value": round(main_run["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
        "impl": "ours",
        "config": {"model": "GPT-J-6B sizes", "n_layer": n_layer, "n_layer_full": GPTJ_6B["n_layer"],
                   "n_embd": cfg.n_embd, "n_head": cfg.n_head, "head_dim": cfg.head_dim,
                   "rotary_dim": cfg.rotary, "n_inner": cfg.inner, "vocab_size": V,
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
            r = decode_run(b, min(args.steps, 32), max(3, min(args.warmup, 4)))
            points[name] = round(r["tok_s"], 2)
            points[name + "_hbm_frac"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        line["points"] = points

        # prefill: one 2,048-token prompt, time to the logits of its last position
        T = 2048
        engine = qs.Engine(model, max_tokens=T, max_batch=1, max_context=T)
        prompt = [int(t) for t in rng.integers(0, V, T)]
        times = []
        for i in range(5):
            slot = engine.acquire()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            engine.step([slot], [prompt])
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            engine.release(slot)
        ms = sorted(times[2:])[len(times[2:]) // 2]
        D, F, H, dh = cfg.n_embd, cfg.inner, cfg.n_head, cfg.head_dim
        flops = n_layer * (2 * T * D * (3 * D) + 2 * T * D * D + 2 * 2 * T * D * F
                           + 2 * 2 * dh * H * T * (T + 1) / 2) + 2 * D * V
        line["prefill"] = {"value": round(T * 1000.0 / ms, 1), "tokens": T, "ms": round(ms, 3),
                           "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        del engine
        torch.cuda.empty_cache()

        # end to end: the Python entry point, host token lists in and out, every step copies the
        # step's metadata from pinned host memory and reads the chosen tokens back
        steps = 2 * args.steps                          # twice the steps: the prefill before them leaves the GPU power-capped for a while
        engine = qs.Engine(model, max_tokens=args.batch * ctx, max_batch=args.batch, max_context=ctx)
        prompt_len = ctx - steps - 4
        prompts = [[int(t) for t in rng.integers(0, V, prompt_len)] for _ in range(args.batch)]
        qs.generate(engine, [p[:64] for p in prompts], max_new_tokens=4, sampling=qs.SamplingConfig.greedy(),
                    stop_tokens=())
        t0 = sampler.mark()
        res = qs.generate(engine, prompts, max_new_tokens=steps + 1, sampling=qs.SamplingConfig.greedy(),
                          stop_tokens=())
        t1 = sampler.mark()
        assert all(len(t) == steps + 1 for t in res.tokens)
        rows = args.batch
        line["e2e"] = {"value": round(res.decode_tokens / res.decode_seconds, 2), "unit": "tokens/s",
                       "h2d_bytes_per_step": (7 * rows + 1) * 4, "d2h_bytes_per_step": rows * 4,
                       "prefill_tok_s": round(res.prefill_tokens / res.prefill_seconds, 1),
                       "clocks": sampler.summary(t0, t1)}
    sampler.stop()
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
