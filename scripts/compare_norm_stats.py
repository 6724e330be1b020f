#!/usr/bin/env python
"""Layer-wise absolute / relative difference of two ``norm_stats.json`` files
(reference: scripts/compare_norm_stats.py:17-86)."""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np


def compare(a: dict, b: dict) -> list:
    rows = []
    for layer in sorted(set(a) & set(b), key=lambda s: int(s)):
        for side in ("inputs", "targets"):
            for stat in ("mean", "std"):
                x, y = np.asarray(a[layer][side][stat], dtype=np.float64), np.asarray(b[layer][side][stat], dtype=np.float64)
                if x.shape != y.shape:
                    rows.append((layer, side, stat, float("nan"), float("nan"), "shape mismatch"))
                    continue
                diff = np.abs(x - y)
                rel = diff / (np.abs(x) + 1e-12)
                rows.append((layer, side, stat, float(diff.max()), float(rel.mean()), ""))
    missing = sorted(set(a) ^ set(b))
    return rows, missing


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("file_a")
    ap.add_argument("file_b")
    ap.add_argument("--tolerance", type=float, default=None, help="exit 1 if any max abs diff exceeds this")
    args = ap.parse_args(argv)
    with open(args.file_a) as fa, open(args.file_b) as fb:
        rows, missing = compare(json.load(fa), json.load(fb))
    print(f"{'layer':>5} {'side':>8} {'stat':>5} {'max_abs_diff':>14} {'mean_rel_diff':>14}")
    worst = 0.0
    for layer, side, stat, mx, rel, note in rows:
        print(f"{layer:>5} {side:>8} {stat:>5} {mx:14.6g} {rel:14.6g} {note}")
        if mx == mx:
            worst = max(worst, mx)
    if missing:
        print("layers present in only one file:", ", ".join(missing))
    return 1 if (args.tolerance is not None and worst > args.tolerance) else 0


if __name__ == "__main__":
    sys.exit(main())
