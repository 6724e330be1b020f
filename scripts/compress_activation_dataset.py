#!/usr/bin/env python
"""Re-write an activation dataset with compressed chunks (reference: scripts/compress_activation_dataset.py:78-196).

The reference copies HDF5 chunks into Zarr/Blosc-lz4 stores that nothing in its code base can read back.  This
tool keeps the dataset readable by every store of this framework: ``--format hdf5-gzip`` rewrites each chunk with
deflate-compressed HDF5 chunks (same manifest, metadata and norm stats); ``--format zarr`` is offered only when the
optional ``zarr`` package is installed.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from crosslayer_coding_b200.io import hdf5, manifest  # noqa: E402


def compress(src: str, dst: str, fmt: str = "hdf5-gzip", chunk_rows: int = 16384) -> str:
    meta = manifest.load_metadata(src)
    sizes = manifest.read_index(os.path.join(src, "index.bin"), meta["total_tokens"])
    os.makedirs(dst, exist_ok=True)
    for cid in sorted(sizes):
        with hdf5.open_chunk(src, cid) as f:
            layers = {}
            for i, name in enumerate(f.layer_groups()):
                layers[int(name.split("_")[1])] = (f[f"{name}/inputs"].read_all(), f[f"{name}/targets"].read_all())
        if fmt == "hdf5-gzip":
            hdf5.write_chunk_file(os.path.join(dst, f"chunk_{cid}.hdf5"), layers, compression="gzip", chunk_rows=min(chunk_rows, sizes[cid]))
        else:
            import zarr  # optional

            root = zarr.open(os.path.join(dst, f"chunk_{cid}.zarr"), mode="w")
            for l, (x, y) in layers.items():
                g = root.create_group(f"layer_{l}")
                g.create_dataset("inputs", data=x, chunks=(min(chunk_rows, len(x)), x.shape[1]))
                g.create_dataset("targets", data=y, chunks=(min(chunk_rows, len(y)), y.shape[1]))
    for name in ("index.bin", "metadata.json", "norm_stats.json"):
        if os.path.exists(os.path.join(src, name)):
            shutil.copy(os.path.join(src, name), os.path.join(dst, name))
    return dst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input-dir", required=True)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--format", choices=["hdf5-gzip", "zarr"], default="hdf5-gzip")
    ap.add_argument("--chunk-rows", type=int, default=16384)
    args = ap.parse_args(argv)
    print(compress(args.input_dir, args.output_dir, args.format, args.chunk_rows))
    return 0


if __name__ == "__main__":
    sys.exit(main())
