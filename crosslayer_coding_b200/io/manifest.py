"""``index.bin`` manifest, ``metadata.json`` and ``norm_stats.json`` of an activation dataset.

``index.bin`` exists in two layouts (reference: clt/activation_generation/generator.py:914-925 writes the
first, clt/training/data/local_activation_store.py:93-172 reads both):

* 3-field, one record per chunk: ``int32 chunk_id, int32 num_tokens, int64 offset`` (16 bytes);
* legacy 2-field, one record per row: ``uint32 chunk_id, uint32 row_id`` (8 bytes).

The reader tries the 3-field layout when the size is a multiple of 16 and accepts it only if the token
counts add up to ``metadata.total_tokens``; otherwise it falls back to the legacy layout.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterable, List, Optional, Tuple

import numpy as np

REC3 = np.dtype([("chunk_id", "<i4"), ("num_tokens", "<i4"), ("offset", "<i8")])
REC2 = np.dtype([("chunk_id", "<u4"), ("row_id", "<u4")])


def write_index_3field(path: str, records: Iterable[Tuple[int, int, int]]) -> None:
    arr = np.array(list(records), dtype=REC3)
    tmp = path + ".tmp"
    arr.tofile(tmp)
    os.replace(tmp, path)


def write_index_legacy(path: str, pairs: np.ndarray) -> None:
    arr = np.ascontiguousarray(pairs, dtype=np.uint32).reshape(-1, 2)
    tmp = path + ".tmp"
    arr.tofile(tmp)
    os.replace(tmp, path)


def parse_index_bytes(raw: bytes, total_tokens: Optional[int] = None) -> Dict[int, int]:
    """``{chunk_id: rows}`` from the bytes of an ``index.bin`` in either layout."""
    n = len(raw)
    if n == 0:
        raise ValueError("empty manifest")
    if n % 16 == 0:
        rec = np.frombuffer(raw, dtype=REC3)
        ok = bool(np.all(rec["num_tokens"] > 0)) and bool(np.all(rec["chunk_id"] >= 0))
        if ok and total_tokens is not None:
            ok = int(rec["num_tokens"].astype(np.int64).sum()) == int(total_tokens)
        if ok and total_tokens is None:
            # without metadata: offsets must be the running sum of the token counts
            off = np.concatenate([[0], np.cumsum(rec["num_tokens"].astype(np.int64))[:-1]])
            ok = bool(np.array_equal(off, rec["offset"]))
        if ok:
            return {int(c): int(t) for c, t in zip(rec["chunk_id"], rec["num_tokens"])}
    if n % 8 != 0:
        raise ValueError(f"manifest size {n} is neither a multiple of 16 nor of 8 bytes")
    pairs = np.frombuffer(raw, dtype=REC2)
    if pairs.size == 0:
        raise ValueError("empty manifest")
    ids, counts = np.unique(pairs["chunk_id"], return_counts=True)
    # rows per chunk = highest row id + 1 when rows are listed completely, else the count
    sizes: Dict[int, int] = {}
    max_row = np.zeros(int(ids.max()) + 1, dtype=np.int64)
    np.maximum.at(max_row, pairs["chunk_id"], pairs["row_id"].astype(np.int64))
    for c, k in zip(ids, counts):
        sizes[int(c)] = max(int(k), int(max_row[int(c)]) + 1)
    return sizes


def read_index(path: str, total_tokens: Optional[int] = None) -> Dict[int, int]:
    with open(path, "rb") as fh:
        return parse_index_bytes(fh.read(), total_tokens)


def load_metadata(dataset_dir: str) -> Dict[str, Any]:
    with open(os.path.join(dataset_dir, "metadata.json")) as fh:
        meta = json.load(fh)
    for key in ("num_layers", "d_model", "total_tokens"):
        if key not in meta:
            raise ValueError(f"metadata.json misses required key {key!r}")
    return meta


def load_norm_stats(dataset_dir: str) -> Optional[Dict[str, Any]]:
    path = os.path.join(dataset_dir, "norm_stats.json")
    if not os.path.exists(path):
        return None
    with open(path) as fh:
        return json.load(fh)
