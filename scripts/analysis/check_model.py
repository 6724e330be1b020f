#!/usr/bin/env python
"""Print what a checkpoint contains: tensor names, shapes, dtypes, norms and simple sanity flags
(reference: scripts/analysis/check_model.py, an ad-hoc state-dict poke).

    python scripts/analysis/check_model.py path/to/model.safetensors [--config cfg.json]
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("checkpoint")
    ap.add_argument("--config", default=None)
    args = ap.parse_args()
    if args.checkpoint.endswith(".safetensors"):
        from safetensors.torch import load_file

        sd = load_file(args.checkpoint)
    else:
        sd = torch.load(args.checkpoint, map_location="cpu", weights_only=False)
        sd = sd.get("model_state_dict", sd) if isinstance(sd, dict) else sd
    if args.config:
        cfg = json.load(open(args.config))
        print("config:", {k: cfg[k] for k in ("num_layers", "num_features", "d_model", "activation_fn", "decoder_tying") if k in cfg})
    total = 0
    for name in sorted(sd):
        t = sd[name]
        if not torch.is_tensor(t):
            continue
        total += t.numel()
        f = t.float()
        flags = []
        if not torch.isfinite(f).all():
            flags.append("NON-FINITE")
        if f.numel() and float(f.abs().max()) == 0.0:
            flags.append("all zero")
        print(f"{name:60s} {str(tuple(t.shape)):24s} {str(t.dtype):16s} |x| mean {float(f.abs().mean()):.3e} max {float(f.abs().max()):.3e} {' '.join(flags)}")
    print(f"{total:,} parameters")
    return 0


if __name__ == "__main__":
    sys.exit(main())
