"""Trace replay: feed given token ids through a model step by step and write logits.

Nothing is sampled.  The program drives the library's own model, step function, cache
and kernels; it has no forward pass, cache or loader of its own.  See `bin/trace_run`.

Input (standard input, one JSON object a line):
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` holds the logits at the wanted
places, in the order of the entries and of `want`, little-endian float32 [wanted, vocab].
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--max-batch", type=int, default=0, help="most live requests (default: what the cache allows)")
    args = ap.parse_args(argv)

    print("[qstream] trace_run: loading the library (the kernels are compiled at the first call) ...",
          file=sys.stderr, flush=True)
    import torch
    from .csrc import ops
    from .engine import Engine, load_model
    from .errors import QStreamError

    if not torch.cuda.is_available():
        print("[qstream] trace_run: no CUDA device; the library has no CPU path", file=sys.stderr)
        return 2
    try:
        ops.library()
        model = load_model(args.model, dtype=args.dtype, device="cuda")
        page = 64
        max_tokens = max(page, -(-args.max_tokens // page) * page)
        max_batch = args.max_batch or max(1, max_tokens // page)
        engine = Engine(model, max_tokens=max_tokens, max_batch=max_batch)
    except QStreamError as e:
        print(str(e), file=sys.stderr)
        return 1
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    print("[qstream] trace_run: ready", file=sys.stderr, flush=True)

    slot_of: dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step_no = rec["step"]
            entries = rec.get("entries", [])
            ids = [str(e["id"]) for e in entries]
            for rid in ids:
                if rid not in slot_of:
                    slot_of[rid] = engine.acquire()
            slots = [slot_of[rid] for rid in ids]
            tokens = [list(e["tokens"]) for e in entries]
            want = [list(e.get("want", [])) for e in entries]
            logits = engine.step(slots, tokens, want) if entries else None
            if logits is not None and logits.shape[0] > 0:
                host = logits.to("cpu", torch.float32).contiguous().numpy()
                engine.check_status()
                host.astype("<f4", copy=False).tofile(out_dir / f"{step_no}.f32")
            else:
                engine.check_status()
            for rid in rec.get("end", []):
                rid = str(rid)
                if rid in slot_of:
                    engine.release(slot_of.pop(rid))
        except QStreamError as e:
            print(str(e), file=sys.stderr, flush=True)
            return 1
        except (KeyError, TypeError, ValueError) as e:
            print(f"[qstream] trace_run: bad step record: {e!r}: {line[:200]}", file=sys.stderr, flush=True)
            return 1
        print(f"done {step_no}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
