#!/usr/bin/env python
"""Globally shuffle the rows of a manifest dataset into new fixed-size chunks
(reference: scripts/scramble_dataset.py:91-292).

Every output chunk draws its rows from all input chunks; the same row permutation is applied to every layer and
to inputs and targets.  The output gets a legacy 2-field ``index.bin``, a copy of ``norm_stats.json`` and
``metadata.json`` extended with ``scrambled_from`` / ``scramble_seed``.  Rows are gathered per input chunk with
the native HDF5 reader (sorted row reads), not one row at a time.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from crosslayer_coding_b200.io import hdf5, manifest  # noqa: E402


def scramble(src: str, dst: str, chunk_tokens: int, seed: int = 0, compression=None) -> str:
    meta = manifest.load_metadata(src)
    sizes = manifest.read_index(os.path.join(src, "index.bin"), meta["total_tokens"])
    pairs = np.concatenate([np.stack([np.full(n, c, dtype=np.uint32), np.arange(n, dtype=np.uint32)], axis=1) for c, n in sorted(sizes.items())])
    rng = np.random.default_rng(seed)
    pairs = pairs[rng.permutation(len(pairs))]
    os.makedirs(dst, exist_ok=True)
    L, d = int(meta["num_layers"]), int(meta["d_model"])
    files = {c: hdf5.open_chunk(src, c) for c in sizes}
    names = {c: f.layer_groups() for c, f in files.items()}
    new_pairs = []
    for out_id, start in enumerate(range(0, len(pairs), chunk_tokens)):
        part = pairs[start : start + chunk_tokens]
        n = len(part)
        layers = {}
        for l in range(L):
            sample = files[int(part[0, 0])][f"{names[int(part[0, 0])][l]}/inputs"]
            x = np.empty((n, d), dtype=sample.dtype)
            y = np.empty((n, d), dtype=sample.dtype)
            for c in np.unique(part[:, 0]):
                pos = np.nonzero(part[:, 0] == c)[0]
                rows = part[pos, 1].astype(np.int64)
                order = np.argsort(rows, kind="stable")
                x[pos[order]] = files[int(c)][f"{names[int(c)][l]}/inputs"].read_rows(rows[order])
                y[pos[order]] = files[int(c)][f"{names[int(c)][l]}/targets"].read_rows(rows[order])
            layers[l] = (x, y)
        hdf5.write_chunk_file(os.path.join(dst, f"chunk_{out_id}.h5"), layers, compression=compression)
        new_pairs.append(np.stack([np.full(n, out_id, dtype=np.uint32), np.arange(n, dtype=np.uint32)], axis=1))
    for f in files.values():
        f.close()
    manifest.write_index_legacy(os.path.join(dst, "index.bin"), np.concatenate(new_pairs))
    meta = dict(meta, chunk_tokens=int(chunk_tokens), scrambled_from=os.path.abspath(src), scramble_seed=int(seed))
    with open(os.path.join(dst, "metadata.json"), "w") as fh:
        json.dump(meta, fh, indent=2)
    if os.path.exists(os.path.join(src, "norm_stats.json")):
        shutil.copy(os.path.join(src, "norm_stats.json"), os.path.join(dst, "norm_stats.json"))
    return dst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input-dir", required=True)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--chunk-tokens", type=int, default=None, help="rows per output chunk (default: as in the source metadata)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--compression", default=None)
    args = ap.parse_args(argv)
    meta = manifest.load_metadata(args.input_dir)
    chunk = args.chunk_tokens or int(meta.get("chunk_tokens", 0)) or 100_000
    print(scramble(args.input_dir, args.output_dir, chunk, args.seed, args.compression))
    return 0


if __name__ == "__main__":
    sys.exit(main())
