"""`qs-mkmodel`: write a model folder with random weights from a configuration and a seed.

    qs-mkmodel --config config.json --seed 0 --out DIR [--dtype bfloat16|float32]
               [--matrix-std 0.02] [--norm-spread 0.1] [--bias-std 0.02] [--device cpu|cuda]

The folder holds `config.json` and `model.safetensors` and loads like any checkpoint.  The weights
are a function of the seed and of each tensor's name (weights/random_init.py): the same command gives
the same file on any machine, made by the host or by the device kernel, and
`CausalLM.random(config, seed)` holds the same values without a file.  QStream has no such tool; it
exists so that every path, the loader included, can be exercised without a checkpoint.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="qs-mkmodel", description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", required=True, help="a config.json with the architecture's own keys")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True, help="folder to write")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--matrix-std", type=float, default=0.02)
    ap.add_argument("--norm-spread", type=float, default=0.1)
    ap.add_argument("--bias-std", type=float, default=0.02)
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"], help="where the values are made")
    args = ap.parse_args(argv)

    from .config import config_from_dict
    from .errors import QStreamError
    from .weights import InitScales, write_model_folder
    try:
        with open(args.config) as fh:
            cfg = config_from_dict(json.load(fh))
        folder = write_model_folder(args.out, cfg, args.seed, args.dtype,
                                    InitScales(args.matrix_std, args.norm_spread, args.bias_std), args.device)
    except (OSError, ValueError) as e:
        print(f"qs-mkmodel: {e}", file=sys.stderr)
        return 1
    except QStreamError as e:
        print(str(e), file=sys.stderr)
        return 1
    print(folder)
    return 0


if __name__ == "__main__":
    sys.exit(main())
