"""``llmserve_b200 random-model``: write config.json and model.safetensors from sizes and a seed."""

from __future__ import annotations

import argparse
import json


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(prog="llmserve_b200 random-model")
    ap.add_argument("out", help="folder to write")
    g = ap.add_mutually_exclusive_group(required=True)
    g.add_argument("--preset", help="a size preset, e.g. smollm2-135m")
    g.add_argument("--config", help="a config.json to take the sizes from")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    args = ap.parse_args(argv)

    import torch

    from .config.registry import architecture_for
    from .models.hub import preset_config_dict
    from .weights import write_random_model

    d = preset_config_dict(args.preset) if args.preset else json.load(open(args.config))
    cfg = architecture_for(d).config_cls.from_dict(d)
    write_random_model(args.out, cfg, args.seed, getattr(torch, args.store_dtype))
    print(f"wrote {args.out} ({cfg.num_parameters():,} parameters, seed {args.seed})")


if __name__ == "__main__":
    main()
