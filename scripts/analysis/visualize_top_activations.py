#!/usr/bin/env python
"""Render the JSON shards written by ``collect_top_activations.py`` as a static HTML page: for every feature its
top sequences with tokens shaded by activation (reference: scripts/analysis/visualize_top_activations.py, which
does the same inside a notebook with plotly colour scales and ipywidgets; this version has no dependencies).

    python scripts/analysis/visualize_top_activations.py --input-dir top/ --output top.html [--features 0 5 9]
"""
from __future__ import annotations

import argparse
import glob
import html
import json
import os
import sys


def shade(value: float, vmax: float) -> str:
    a = 0.0 if vmax <= 0 else max(0.0, min(1.0, value / vmax))
    return f"background-color: rgba(255, 120, 0, {a:.3f})"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input-dir", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--features", type=int, nargs="*", default=None)
    ap.add_argument("--max-features", type=int, default=200)
    args = ap.parse_args()
    records = {}
    for path in sorted(glob.glob(os.path.join(args.input_dir, "*.json"))):
        data = json.load(open(path))
        feats = data.get("features", data)
        for fid, items in feats.items():
            records.setdefault(int(fid), []).extend(items)
    wanted = sorted(records) if args.features is None else [f for f in args.features if f in records]
    parts = ["<html><head><meta charset='utf-8'><style>body{font-family:monospace} .tok{padding:1px 2px} h3{margin-bottom:2px}</style></head><body>"]
    for fid in wanted[: args.max_features]:
        items = sorted(records[fid], key=lambda r: -float(r.get("activation", r.get("max_activation", 0.0))))
        parts.append(f"<h3>feature {fid}</h3>")
        for rec in items:
            top = float(rec.get("activation", rec.get("max_activation", 0.0)))
            tokens = rec.get("tokens")
            acts = rec.get("activations")
            if tokens and acts:
                vmax = max(max(acts), 1e-12)
                spans = "".join(f"<span class='tok' style='{shade(a, vmax)}' title='{a:.4f}'>{html.escape(str(t))}</span>" for t, a in zip(tokens, acts))
                parts.append(f"<div>{top:.4f} &nbsp; {spans}</div>")
            else:
                where = {k: rec[k] for k in ("chunk", "row", "token_index", "batch", "position") if k in rec}
                parts.append(f"<div>{top:.4f} &nbsp; {html.escape(json.dumps(where))}</div>")
    parts.append("</body></html>")
    with open(args.output, "w") as f:
        f.write("\n".join(parts))
    print(args.output)
    return 0


if __name__ == "__main__":
    sys.exit(main())
