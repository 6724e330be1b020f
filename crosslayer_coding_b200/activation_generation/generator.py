"""Activation dataset generation (reference: clt/activation_generation/generator.py:468-1058).

``ActivationGenerator(cfg, device).generate_and_save()`` streams ``(inputs, targets)`` dictionaries from an
extractor, keeps per-layer running statistics, and writes a manifest dataset:

* chunks of at least ``chunk_token_threshold`` tokens, rows shuffled with ONE permutation shared by all
  layers of the chunk, datasets ``layer_{id}/inputs|targets`` of shape ``(rows, d)`` row-chunked
  ``(min(rows, 16384), d)``, optional gzip, dtype float32 / float16 / uint16 (bf16 bit patterns);
  ``npz`` as the alternative container;
* ``index.bin`` (3-field records), ``metadata.json``, ``norm_stats.json`` (unbiased std);
* output directory ``{activation_dir}/{model_name}/{basename(dataset_path)}_{split}``;
* optional background upload of every chunk to the activation server with retry classes by HTTP status
  (408/429/5xx retried with exponential backoff and jitter, other 4xx and 507 not), then manifest,
  metadata and norm stats.

Differences: statistics are Chan-merged batch moments in float64 computed with two device reductions per
tensor; chunks are written by the native HDF5 writer (one pass, no reopen-in-append-mode threads); bf16 is
stored by reinterpretation (the reference's value conversion clamps negative numbers to zero).
"""
from __future__ import annotations

import json
import logging
import os
import queue
import random
import threading
import time
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Tuple
from urllib.parse import quote, urljoin

import numpy as np
import torch

from ..config import ActivationConfig
from ..io import hdf5, manifest

logger = logging.getLogger(__name__)

RETRYABLE_STATUS = {408, 429, 500, 502, 503, 504}


class _RunningStat:
    """Mean / M2 of the rows seen so far (Chan's parallel update), float64."""

    def __init__(self, dim: int):
        self.n = 0
        self.mean = np.zeros(dim, dtype=np.float64)
        self.m2 = np.zeros(dim, dtype=np.float64)

    def update(self, x: torch.Tensor) -> None:
        k = int(x.shape[0])
        if k == 0:
            return
        xd = x.double()
        bm = xd.mean(dim=0)
        bm2 = ((xd - bm) ** 2).sum(dim=0)
        bm, bm2 = bm.cpu().numpy(), bm2.cpu().numpy()
        if self.n == 0:
            self.n, self.mean, self.m2 = k, bm, bm2
            return
        tot = self.n + k
        delta = bm - self.mean
        self.mean = self.mean + delta * (k / tot)
        self.m2 = self.m2 + bm2 + delta * delta * (self.n * k / tot)
        self.n = tot

    def finalize(self) -> Tuple[np.ndarray, np.ndarray]:
        var = self.m2 / (self.n - 1) if self.n > 1 else np.zeros_like(self.m2)
        return self.mean, np.sqrt(np.maximum(var, 0.0))


class PerformanceProfiler:
    """Wall-clock timings of named generation phases plus process memory (reference generator.py:59-211)."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self.timings: Dict[str, List[float]] = {}

    def measure(self, name: str):
        prof = self

        class _Ctx:
            def __enter__(self):
                self.t0 = time.perf_counter()
                return self

            def __exit__(self, *exc):
                if prof.enabled:
                    prof.timings.setdefault(name, []).append(time.perf_counter() - self.t0)

        return _Ctx()

    def log_system_metrics(self, tag: str = "") -> Dict[str, float]:
        out: Dict[str, float] = {}
        try:
            import psutil

            p = psutil.Process()
            out = {"rss_gb": p.memory_info().rss / 1e9, "cpu_percent": psutil.cpu_percent(interval=None)}
        except Exception:  # psutil is optional
            pass
        if torch.cuda.is_available():
            out["cuda_allocated_gb"] = torch.cuda.memory_allocated() / 1e9
        if self.enabled and out:
            logger.info("system metrics %s: %s", tag, out)
        return out

    def report(self) -> None:
        if not self.enabled:
            return
        for name, vals in sorted(self.timings.items(), key=lambda kv: -sum(kv[1])):
            logger.info("generation phase %-24s total %8.2fs  n=%d  avg %.4fs", name, sum(vals), len(vals), sum(vals) / len(vals))


def dataset_id_for(cfg: ActivationConfig) -> str:
    return f"{cfg.model_name}/{os.path.basename(cfg.dataset_path)}_{cfg.dataset_split}"


def upload_file_with_retries(session, url: str, path: Path, field: str, cfg: ActivationConfig, content_type: str,
                             sleep=time.sleep) -> bool:
    """POST one file as multipart; retry 408/429/5xx and transport errors with exponential backoff + jitter."""
    import requests

    retries = max(1, cfg.upload_max_retries)
    for attempt in range(retries):
        retryable = False
        try:
            with open(path, "rb") as fh:
                resp = session.post(url, files={field: (path.name, fh, content_type)},
                                    headers={"X-Num-Tokens": str(cfg.chunk_token_threshold), "X-Saved-Dtype": cfg.activation_dtype},
                                    timeout=300)
            if resp.ok:
                return True
            if resp.status_code in RETRYABLE_STATUS:
                retryable = True
                logger.warning("upload of %s: status %d (attempt %d/%d)", path.name, resp.status_code, attempt + 1, retries)
            else:
                logger.error("upload of %s failed with status %d; not retrying", path.name, resp.status_code)
        except requests.exceptions.RequestException as exc:
            retryable = True
            logger.warning("upload of %s: %s (attempt %d/%d)", path.name, exc, attempt + 1, retries)
        except Exception as exc:  # noqa: BLE001 - programming errors are not retried
            logger.error("upload of %s raised %s; not retrying", path.name, exc)
        if not retryable:
            return False
        if attempt + 1 < retries:
            back = min(cfg.upload_initial_backoff * (2 ** attempt), cfg.upload_max_backoff)
            sleep(back + random.uniform(-0.1 * back, 0.1 * back))
    return False


def _async_uploader(upload_q: "queue.Queue[Optional[Path]]", cfg: ActivationConfig) -> None:
    import requests

    if cfg.remote_server_url is None:
        while True:
            item = upload_q.get()
            upload_q.task_done()
            if item is None:
                return
    base = cfg.remote_server_url.rstrip("/") + "/"
    did = quote(dataset_id_for(cfg), safe="")
    session = requests.Session()
    while True:
        p = upload_q.get()
        try:
            if p is None:
                return
            idx = int(p.stem.split("_")[-1])
            ok = upload_file_with_retries(session, urljoin(base, f"datasets/{did}/chunks/{idx}"), p, "chunk_file", cfg, "application/x-hdf5")
            if ok and cfg.delete_after_upload:
                try:
                    p.unlink(missing_ok=True)
                except OSError as exc:
                    logger.warning("could not delete %s after upload: %s", p, exc)
            if not ok:
                logger.error("chunk %s stays local: upload failed", p.name)
        finally:
            upload_q.task_done()


class ActivationGenerator:
    def __init__(self, cfg: ActivationConfig, device: Optional[Any] = None, extractor: Optional[Any] = None):
        self.cfg = cfg
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.torch_dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[cfg.activation_dtype]
        self.profiler = PerformanceProfiler(enabled=cfg.enable_profiling)
        if extractor is None:
            from .extractor import ActivationExtractorCLT

            extractor = ActivationExtractorCLT(
                model_name=cfg.model_name, mlp_input_module_path_template=cfg.mlp_input_module_path_template,
                mlp_output_module_path_template=cfg.mlp_output_module_path_template, device=self.device,
                model_dtype=cfg.model_dtype, context_size=cfg.context_size, inference_batch_size=cfg.inference_batch_size,
                exclude_special_tokens=cfg.exclude_special_tokens, prepend_bos=cfg.prepend_bos,
                nnsight_tracer_kwargs=cfg.nnsight_tracer_kwargs, nnsight_invoker_args=cfg.nnsight_invoker_args,
            )
        self.extractor = extractor
        ds_name = os.path.basename(cfg.dataset_path)
        self.out_dir = Path(cfg.activation_dir) / cfg.model_name / f"{ds_name}_{cfg.dataset_split}"
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.storage_type = "local"
        self._upload_q: Optional["queue.Queue[Optional[Path]]"] = None
        self._uploader: Optional[threading.Thread] = None
        self.manifest_rows: List[Tuple[int, int, int]] = []

    # ------------------------------------------------------------------ storage selection
    def set_storage_type(self, storage_type: str) -> None:
        st = storage_type.lower()
        if st not in ("local", "remote"):
            raise ValueError(f"Unknown storage type: {storage_type}")
        if st == "remote" and not self.cfg.remote_server_url:
            logger.warning("storage type 'remote' without remote_server_url: chunks stay local")
        self.storage_type = st
        if st == "remote" and self.cfg.remote_server_url and self._uploader is None:
            self._upload_q = queue.Queue()
            self._uploader = threading.Thread(target=_async_uploader, args=(self._upload_q, self.cfg), daemon=True)
            self._uploader.start()

    # ------------------------------------------------------------------ main loop
    def generate_and_save(self) -> None:
        cfg = self.cfg
        stream = self.extractor.stream_activations(
            dataset_path=cfg.dataset_path, dataset_split=cfg.dataset_split, dataset_text_column=cfg.dataset_text_column,
            streaming=cfg.streaming, dataset_trust_remote_code=cfg.dataset_trust_remote_code, cache_path=cfg.cache_path,
        )
        buf_in: Dict[int, List[torch.Tensor]] = {}
        buf_tg: Dict[int, List[torch.Tensor]] = {}
        stats: Dict[int, Dict[str, _RunningStat]] = {}
        layer_ids: Optional[List[int]] = None
        d_model = -1
        buffered = total = 0
        chunk_idx = 0
        offset = 0
        target = cfg.target_total_tokens
        for inputs, targets in stream:
            if not inputs:
                continue
            if layer_ids is None:
                layer_ids = sorted(inputs.keys())
                d_model = int(inputs[layer_ids[0]].shape[-1])
                for l in layer_ids:
                    buf_in[l], buf_tg[l] = [], []
                    if cfg.compute_norm_stats:
                        stats[l] = {"inputs": _RunningStat(d_model), "targets": _RunningStat(d_model)}
            n = int(inputs[layer_ids[0]].shape[0])
            if n == 0:
                continue
            if target is not None and total + n > target:
                n = int(target - total)
            with self.profiler.measure("accumulate"):
                for l in layer_ids:
                    x, y = inputs[l][:n].detach(), targets[l][:n].detach()
                    buf_in[l].append(x)
                    buf_tg[l].append(y)
                    if cfg.compute_norm_stats:
                        stats[l]["inputs"].update(x)
                        stats[l]["targets"].update(y)
            buffered += n
            total += n
            if buffered >= cfg.chunk_token_threshold:
                with self.profiler.measure("write_chunk"):
                    rows = self._write_chunk(chunk_idx, buf_in, buf_tg, layer_ids, offset)
                offset += rows
                chunk_idx += 1
                buffered = 0
                for l in layer_ids:
                    buf_in[l].clear()
                    buf_tg[l].clear()
            if target is not None and total >= target:
                break
        if layer_ids is None:
            raise RuntimeError("the extractor yielded no activations")
        if buffered > 0:
            rows = self._write_chunk(chunk_idx, buf_in, buf_tg, layer_ids, offset)
            offset += rows
            chunk_idx += 1
        manifest.write_index_3field(str(self.out_dir / "index.bin"), self.manifest_rows)
        meta = {
            "model_name": cfg.model_name, "dataset": cfg.dataset_path, "split": cfg.dataset_split,
            "num_layers": len(layer_ids), "d_model": d_model, "dtype": cfg.activation_dtype,
            "total_tokens": int(total), "chunk_tokens": int(cfg.chunk_token_threshold),
            "created": time.strftime("%Y-%m-%dT%H:%M:%S"),
        }
        with open(self.out_dir / "metadata.json", "w") as fh:
            json.dump(meta, fh, indent=2)
        norm: Optional[Dict[str, Any]] = None
        if cfg.compute_norm_stats:
            norm = {}
            for l in layer_ids:
                mi, si = stats[l]["inputs"].finalize()
                mt, st = stats[l]["targets"].finalize()
                norm[str(l)] = {"inputs": {"mean": mi.tolist(), "std": si.tolist()}, "targets": {"mean": mt.tolist(), "std": st.tolist()}}
            with open(self.out_dir / "norm_stats.json", "w") as fh:
                json.dump(norm, fh)
        if self._upload_q is not None:
            self._upload_q.put(None)
            self._upload_q.join()
            self._upload_sidecars(meta, norm)
        self.profiler.report()
        logger.info("wrote %d tokens in %d chunks to %s", total, chunk_idx, self.out_dir)

    # ------------------------------------------------------------------ chunk writer
    def _write_chunk(self, chunk_idx: int, buf_in, buf_tg, layer_ids: List[int], offset: int) -> int:
        cfg = self.cfg
        first = torch.cat(buf_in[layer_ids[0]], dim=0)
        rows = int(first.shape[0])
        perm = torch.randperm(rows, device=first.device)  # one permutation for every layer of the chunk
        layers: Dict[int, Tuple[np.ndarray, np.ndarray]] = {}
        for l in layer_ids:
            x = first if l == layer_ids[0] else torch.cat(buf_in[l], dim=0)
            y = torch.cat(buf_tg[l], dim=0)
            layers[l] = (hdf5.to_storage_array(x[perm], cfg.activation_dtype), hdf5.to_storage_array(y[perm], cfg.activation_dtype))
        if cfg.output_format == "hdf5":
            path = self.out_dir / f"chunk_{chunk_idx}.hdf5"
            hdf5.write_chunk_file(str(path), layers, compression=cfg.compression if cfg.compression in ("gzip",) else None)
        else:
            path = self.out_dir / f"chunk_{chunk_idx}.npz"
            flat = {}
            for l, (x, y) in layers.items():
                flat[f"layer_{l}_inputs"], flat[f"layer_{l}_targets"] = x, y
            (np.savez_compressed if cfg.compression else np.savez)(str(path), **flat)
        self.manifest_rows.append((chunk_idx, rows, offset))
        if self._upload_q is not None and cfg.output_format == "hdf5":
            self._upload_q.put(path)
        return rows

    # ------------------------------------------------------------------ sidecar uploads
    def _upload_sidecars(self, meta: Dict[str, Any], norm: Optional[Dict[str, Any]]) -> None:
        import requests

        cfg = self.cfg
        if not cfg.remote_server_url:
            return
        base = cfg.remote_server_url.rstrip("/") + "/"
        did = quote(dataset_id_for(cfg), safe="")
        session = requests.Session()
        upload_file_with_retries(session, urljoin(base, f"datasets/{did}/manifest"), self.out_dir / "index.bin", "manifest_file", cfg,
                                 "application/octet-stream")
        self._upload_json(session, urljoin(base, f"datasets/{did}/metadata"), meta)
        if norm is not None:
            self._upload_json(session, urljoin(base, f"datasets/{did}/norm_stats"), norm)

    def _upload_json(self, session, url: str, payload: Dict[str, Any]) -> bool:
        import requests

        cfg = self.cfg
        for attempt in range(max(1, cfg.upload_max_retries)):
            try:
                resp = session.post(url, json=payload, timeout=120)
                if resp.ok:
                    return True
                if resp.status_code not in RETRYABLE_STATUS:
                    logger.error("JSON upload to %s failed with status %d", url, resp.status_code)
                    return False
            except requests.exceptions.RequestException as exc:
                logger.warning("JSON upload to %s: %s", url, exc)
            time.sleep(min(cfg.upload_initial_backoff * (2 ** attempt), cfg.upload_max_backoff))
        return False


def main(argv: Optional[List[str]] = None) -> None:
    """``python -m crosslayer_coding_b200.activation_generation.generator --config cfg.yaml``"""
    import argparse

    import yaml

    ap = argparse.ArgumentParser(description="Generate an activation dataset from a YAML ActivationConfig")
    ap.add_argument("--config", required=True)
    ap.add_argument("--device", default=None)
    ap.add_argument("--storage-type", default="local", choices=["local", "remote"])
    args = ap.parse_args(argv)
    with open(args.config) as fh:
        cfg = ActivationConfig(**yaml.safe_load(fh))
    gen = ActivationGenerator(cfg, device=args.device)
    gen.set_storage_type(args.storage_type)
    gen.generate_and_save()


if __name__ == "__main__":
    main()
