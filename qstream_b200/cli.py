"""The `qstream` command line, with QStream's option names (src/main.c:103-130).

    qstream <model_dir> [options]

Options kept with their meaning: -p/--prompt, -n/--max-tokens (256), -t/--temperature (0.7,
0 = greedy), -k/--top-k (40, 0 = off), --top-p (0.9), --repeat-penalty (1.1, 1.0 = off),
--seed (42), --ram-budget MB (here: the cache's share of device memory), --no-mmap,
-v/--verbose (twice for more), -h/--help.  There is no tokenizer in this library, so a
prompt is a list of token ids ("5,17,3"; several requests separated by ';' or given with
repeated -p, or one per line in --prompt-file), and the chat options are gone.  New:
--dtype, --max-batch, --max-ctx, --stop-token (repeatable; "none" for no stop token),
--random-weights SEED with --config FILE (writes nothing; weights are made on the device),
--check-nan (scan every layer's output for values that are not finite, as the reference's
`check_nan` switch does, include/qsf/engine.h:31).
Generated ids go to standard output, one request per line; statistics to standard error as
in src/main.c:323-332.
"""
from __future__ import annotations

import argparse
import json
import signal
import sys
import time


def parse_prompts(args) -> list:
    texts = []
    for p in args.prompt or []:
        texts += [t for t in p.split(";") if t.strip()]
    if args.prompt_file:
        with open(args.prompt_file) as fh:
            texts += [line for line in fh if line.strip()]
    prompts = []
    for t in texts:
        try:
            prompts.append([int(x) for x in t.replace(",", " ").split()])
        except ValueError:
            raise SystemExit(f"Error: a prompt is a list of token ids, got '{t.strip()}'")
    return prompts


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="qstream", description="QStream-B200 - LLM inference on one B200",
                                 formatter_class=argparse.RawDescriptionHelpFormatter, epilog=__doc__)
    ap.add_argument("model", nargs="?", help="model folder (config.json + *.safetensors)")
    ap.add_argument("-p", "--prompt", action="append", help='token ids, e.g. "5,17,3" (";" separates requests)')
    ap.add_argument("--prompt-file", help="file with one request (token ids) per line")
    ap.add_argument("-n", "--max-tokens", type=int, default=256, help="max tokens to generate (default: 256)")
    ap.add_argument("-t", "--temperature", type=float, default=0.7, help="sampling temperature (default: 0.7, 0=greedy)")
    ap.add_argument("-k", "--top-k", type=int, default=40, help="top-K sampling (default: 40, 0=disabled)")
    ap.add_argument("--top-p", type=float, default=0.9, help="top-P nucleus sampling (default: 0.9)")
    ap.add_argument("--repeat-penalty", type=float, default=1.1, help="repeat penalty (default: 1.1, 1.0=off)")
    ap.add_argument("--seed", type=int, default=42, help="RNG seed (default: 42)")
    ap.add_argument("--ram-budget", type=int, default=0, help="device memory for the cache in MB (default: auto)")
    ap.add_argument("--no-mmap", action="store_true", help="read the weights instead of mapping them")
    ap.add_argument("-v", "--verbose", action="count", default=0, help="verbose output (use twice for debug)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-batch", type=int, default=64, help="most sequences in a batch (default: 64)")
    ap.add_argument("--max-ctx", type=int, default=0, help="longest sequence (default: the model's)")
    ap.add_argument("--stop-token", action="append", help='stop token id (repeatable); "none" for none; default: eos')
    ap.add_argument("--random-weights", type=int, metavar="SEED", help="random weights instead of a model folder")
    ap.add_argument("--config", help="config.json for --random-weights")
    ap.add_argument("--narrow-fp32", action="store_true",
                    help="with --dtype bfloat16: round matrices stored in 32-bit to bfloat16 (default: they stay 32-bit)")
    ap.add_argument("--check-nan", action="store_true", help="check every layer's output for NaN/Inf (slow)")
    return ap


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.random_weights is None and not args.model:
        print("Error: no model folder specified", file=sys.stderr)
        ap.print_usage(sys.stderr)
        return 1
    prompts = parse_prompts(args)
    if not prompts:
        print("Error: no prompt (-p \"5,17,3\" or --prompt-file)", file=sys.stderr)
        return 1

    import torch
    import qstream_b200 as qs
    from qstream_b200.config import config_from_dict

    try:
        t0 = time.perf_counter()
        if args.random_weights is not None:
            if not args.config:
                print("Error: --random-weights needs --config FILE", file=sys.stderr)
                return 1
            with open(args.config) as fh:
                cfg = config_from_dict(json.load(fh))
            model = qs.CausalLM.random(cfg, args.random_weights, args.dtype, "cuda")
        else:
            model = qs.load_model(args.model, dtype=args.dtype, device="cuda", allow_mmap=not args.no_mmap,
                                  narrow_fp32_matrices=args.narrow_fp32)
        ctx = args.max_ctx or model.spec.max_positions
        max_batch = max(1, min(args.max_batch, len(prompts)))
        max_tokens = max_batch * (-(-min(ctx, model.spec.max_positions) // 64) * 64)
        if args.ram_budget:
            per_token = sum(2 * n.n_kv_heads * n.head_dim for n in model.kv_needs().values()) * \
                torch.empty((), dtype=model.runtime.dtype).element_size()
            max_tokens = min(max_tokens, max(64, args.ram_budget * 2**20 // max(per_token, 1) // 64 * 64))
        engine = qs.Engine(model, qs.EngineConfig(max_tokens=max_tokens, max_batch=max_batch, max_context=ctx,
                                                  verbose=args.verbose, check_nan=args.check_nan))
        if args.verbose:
            print(f"[qstream] model loaded in {(time.perf_counter() - t0) * 1e3:.1f} ms "
                  f"({model.n_parameters / 1e6:.1f} M parameters, {args.dtype})", file=sys.stderr)
        stop = None
        if args.stop_token:
            stop = [] if any(s.lower() == "none" for s in args.stop_token) else [int(s) for s in args.stop_token]
        sampling = qs.SamplingConfig(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                                     repeat_penalty=args.repeat_penalty, seed=args.seed)
        gen = qs.Generator(engine)
        signal.signal(signal.SIGINT, lambda *_: gen.interrupt())        # src/main.c:25-28,260-263
        signal.signal(signal.SIGTERM, lambda *_: gen.interrupt())
        res = gen.generate(prompts, args.max_tokens, sampling, stop)
    except qs.QStreamError as e:
        print(str(e), file=sys.stderr)
        return 1
    for toks in res.tokens:
        print(" ".join(str(t) for t in toks), flush=True)
    n = sum(len(t) for t in res.tokens)
    total = res.prefill_seconds + res.decode_seconds
    print(f"\n--- Stats ---\nRequests: {len(prompts)} in {len(res.batches)} batch(es)\n"
          f"Tokens generated: {n}\nTotal time: {total * 1e3:.1f} ms", file=sys.stderr)
    if res.prefill_seconds > 0:
        print(f"Prefill: {res.prefill_tokens} tokens, {res.prefill_tokens / res.prefill_seconds:.1f} tok/s", file=sys.stderr)
    if res.decode_seconds > 0 and res.decode_tokens:
        print(f"Speed: {res.decode_tokens / res.decode_seconds:.1f} tok/s "
              f"({res.decode_seconds * 1e3 / max(res.decode_tokens, 1):.2f} ms/token)", file=sys.stderr)
    if args.verbose:
        print("Finish reasons: " + " ".join(res.finish_reasons), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
