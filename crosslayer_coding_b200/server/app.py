"""Activation slice server (protocol of the reference: clt_server/core/storage.py:76-253, clt_server/main.py).

Routes:

* ``GET  /api/v1/health`` -> ``{"status": "ok"}``
* ``POST /datasets/{id:path}/chunks/{idx}`` multipart ``chunk_file`` -> stores ``chunk_{idx}.h5`` (201)
* ``POST /datasets/{id:path}/slice?chunk=N`` JSON ``{"rows": [...]}`` -> raw bytes; rows are served in ascending
  order, per layer (numeric layer order) ``inputs`` rows then ``targets`` rows, in the stored dtype
* ``GET  /datasets/{id:path}/info | norm_stats | manifest``
* ``POST /datasets/{id:path}/manifest`` multipart ``manifest_file``; ``POST .../metadata`` and ``.../norm_stats`` JSON (201)

Chunks are read through the native memory-mapped HDF5 reader: a slice gathers exactly the requested rows,
so there is no whole-dataset RAM cache to size (the reference keeps up to 64 full datasets in memory).
Open files sit in an LRU of 128 handles.
"""
from __future__ import annotations

import json
import logging
import threading
from collections import OrderedDict
from pathlib import Path
from typing import Any, Dict, List, Optional

import numpy as np
from fastapi import Body, FastAPI, File, HTTPException, Query, UploadFile
from fastapi.responses import JSONResponse, Response, StreamingResponse
from pydantic import BaseModel

from ..io import hdf5

logger = logging.getLogger(__name__)


class SliceRequest(BaseModel):
    rows: List[int]


class _FileCache:
    def __init__(self, capacity: int = 128):
        self.capacity = capacity
        self._files: "OrderedDict[str, hdf5.H5File]" = OrderedDict()
        self._lock = threading.Lock()

    def get(self, path: Path) -> hdf5.H5File:
        key = str(path)
        with self._lock:
            f = self._files.get(key)
            if f is not None:
                self._files.move_to_end(key)
                return f
            f = hdf5.H5File(key)
            self._files[key] = f
            while len(self._files) > self.capacity:
                _, old = self._files.popitem(last=False)
                old.close()
            return f

    def drop(self, path: Path) -> None:
        with self._lock:
            f = self._files.pop(str(path), None)
            if f is not None:
                f.close()


def create_app(storage_dir: Optional[str] = None) -> FastAPI:
    from .config import settings

    root = Path(storage_dir) if storage_dir is not None else Path(settings.STORAGE_BASE_DIR)
    root.mkdir(parents=True, exist_ok=True)
    cache = _FileCache()
    app = FastAPI(title="CLT Activation Storage Server", version="0.3",
                  description="Stores and serves pre-generated model activations for CLT training.")
    app.state.storage_root = root

    def ds_path(dataset_id: str) -> Path:
        p = (root / dataset_id).resolve()
        if root.resolve() not in p.parents and p != root.resolve():
            raise HTTPException(400, "invalid dataset id")
        return p

    def chunk_file(ds: Path, idx: int) -> Optional[Path]:
        for ext in (".h5", ".hdf5"):
            p = ds / f"chunk_{idx}{ext}"
            if p.exists():
                return p
        return None

    @app.get("/")
    async def read_root():
        return {"message": "Welcome to the CLT Activation Storage Server. See /docs for API details."}

    @app.get("/api/v1/health")
    async def health_check():
        return {"status": "ok"}

    @app.post("/datasets/{dataset_id:path}/chunks/{chunk_idx}", status_code=201)
    async def upload_chunk(dataset_id: str, chunk_idx: int, chunk_file_: UploadFile = File(..., alias="chunk_file")):
        ds = ds_path(dataset_id)
        ds.mkdir(parents=True, exist_ok=True)
        fname = ds / f"chunk_{chunk_idx}.h5"
        tmp = fname.with_suffix(".h5.part")
        with open(tmp, "wb") as fh:
            while True:
                blk = await chunk_file_.read(8 << 20)
                if not blk:
                    break
                fh.write(blk)
        cache.drop(fname)
        tmp.replace(fname)
        logger.info("saved %s (%d bytes)", fname, fname.stat().st_size)
        return {"status": "ok"}

    @app.post("/datasets/{dataset_id:path}/slice")
    async def slice_chunk(dataset_id: str, chunk: int = Query(..., ge=0), request_body: SliceRequest = Body(...)):
        path = chunk_file(ds_path(dataset_id), chunk)
        if path is None:
            raise HTTPException(404, f"Chunk {chunk} not found")
        if not request_body.rows:
            raise HTTPException(400, "rows list in request body cannot be empty")
        try:
            rows = np.sort(np.asarray(request_body.rows, dtype=np.int64))
        except (ValueError, TypeError):
            raise HTTPException(400, "rows must be a list of integers")
        if rows[0] < 0:
            raise HTTPException(400, "rows must be non-negative")
        try:
            f = cache.get(path)
            layers = f.layer_groups()
        except (OSError, KeyError) as exc:
            logger.error("Failed to open %s: %s", path, exc)
            raise HTTPException(500, "Corrupt chunk file")
        if not layers:
            raise HTTPException(500, "No layer groups in chunk")
        try:
            first = f[f"{layers[0]}/inputs"]
            if rows[-1] >= first.rows:
                raise HTTPException(400, f"row index {int(rows[-1])} out of range for chunk with {first.rows} rows")
        except (OSError, KeyError) as exc:
            raise HTTPException(500, f"Missing data in chunk {chunk}: {exc}")

        def iter_layers():
            for name in layers:
                yield f[f"{name}/inputs"].read_rows(rows).tobytes()
                yield f[f"{name}/targets"].read_rows(rows).tobytes()

        return StreamingResponse(iter_layers(), media_type="application/octet-stream")

    def _json_file(dataset_id: str, name: str):
        p = ds_path(dataset_id) / name
        if not p.exists():
            raise HTTPException(404)
        with open(p) as fh:
            return JSONResponse(json.load(fh))

    @app.get("/datasets/{dataset_id:path}/info")
    async def dataset_info(dataset_id: str):
        return _json_file(dataset_id, "metadata.json")

    @app.get("/datasets/{dataset_id:path}/norm_stats")
    async def norm_stats(dataset_id: str):
        return _json_file(dataset_id, "norm_stats.json")

    @app.get("/datasets/{dataset_id:path}/manifest")
    async def manifest(dataset_id: str):
        p = ds_path(dataset_id) / "index.bin"
        if not p.exists():
            raise HTTPException(404)
        return Response(p.read_bytes(), media_type="application/octet-stream")

    @app.post("/datasets/{dataset_id:path}/manifest", status_code=201)
    async def upload_manifest(dataset_id: str, manifest_file: UploadFile = File(...)):
        ds = ds_path(dataset_id)
        ds.mkdir(parents=True, exist_ok=True)
        try:
            content = await manifest_file.read()
            (ds / "index.bin").write_bytes(content)
            return {"status": "ok"}
        except OSError as exc:
            logger.error("Failed to save manifest for %s: %s", dataset_id, exc)
            raise HTTPException(500, "Failed to save manifest")
        finally:
            await manifest_file.close()

    def _save_json(dataset_id: str, name: str, payload: Dict[str, Any]):
        ds = ds_path(dataset_id)
        ds.mkdir(parents=True, exist_ok=True)
        try:
            with open(ds / name, "w") as fh:
                json.dump(payload, fh, indent=2)
        except OSError as exc:
            logger.error("Failed to save %s for %s: %s", name, dataset_id, exc)
            raise HTTPException(500, f"Failed to save {name}")
        return {"status": "ok"}

    @app.post("/datasets/{dataset_id:path}/metadata", status_code=201)
    async def upload_metadata(dataset_id: str, metadata: Dict[str, Any]):
        return _save_json(dataset_id, "metadata.json", metadata)

    @app.post("/datasets/{dataset_id:path}/norm_stats", status_code=201)
    async def upload_norm_stats(dataset_id: str, norm_stats_data: Dict[str, Any]):
        return _save_json(dataset_id, "norm_stats.json", norm_stats_data)

    return app
