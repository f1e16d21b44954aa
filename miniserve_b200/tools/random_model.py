"""Write a model folder (config.json, model.safetensors) with random weights.

    python -m miniserve_b200.tools.random_model --preset tiny-a --seed 0 --out DIR
    python -m miniserve_b200.tools.random_model --config my_config.json --seed 3 --out DIR
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--preset", default=None, help="tiny-a, tiny-b, 0.6b, 1.7b, 8b or 32b")
    ap.add_argument("--config", default=None, help="a config.json to take the sizes from")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="dtype the tensors are stored in")
    ap.add_argument("--std", type=float, default=0.02)
    args = ap.parse_args(argv)
    if (args.preset is None) == (args.config is None):
        ap.error("give exactly one of --preset and --config")

    from ..config.presets import preset
    from ..engine.loader import parse_dtype
    from ..weights.random_init import write_model_folder

    raw = preset(args.preset) if args.preset else json.loads(Path(args.config).read_text())
    print(write_model_folder(args.out, raw, args.seed, dtype=parse_dtype(args.dtype), std=args.std))
    return 0


if __name__ == "__main__":
    sys.exit(main())
