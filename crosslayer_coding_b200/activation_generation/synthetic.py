"""Seeded sparse-dictionary activation generator.

Produces MLP-input / MLP-output pairs with a known sparse structure, so transcoders can be trained,
benchmarked and tested without a language model or a dataset:

* per layer ``l`` a fixed dictionary of ``dict_size`` directions drawn from ``N(0, I/d)`` (unit norm in
  expectation);
* each token's input ``x_l`` is the sum of ``Poisson(active_mean)`` randomly chosen directions with
  ``Exponential(1)`` magnitudes plus ``N(0, input_noise^2)`` noise;
* the output ``y_l = sum_{j<=l} x_j A_{j,l} + N(0, output_noise^2)`` with ``A_{j,l} ~ N(0, a_var/(l+1))``,
  ``a_var = 1/d`` by default, i.e. the cross-layer structure a CLT is built to capture;
* both sides can be standardised per layer with statistics estimated from a calibration sample, which
  are also what ``norm_stats.json`` stores.

The generator is device agnostic (CPU for the small plumbing datasets, GPU for benchmark batches) and
fully determined by ``seed``.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass
from typing import Dict, Iterator, Optional, Tuple

import numpy as np
import torch


@dataclass
class SyntheticSpec:
    num_layers: int
    d_model: int
    dict_size: int
    active_mean: float = 32.0
    input_noise: float = 0.1
    output_noise: float = 0.05
    a_var_scale: Optional[float] = None  # variance of A_{j,l} is a_var_scale/(l+1); default 1/d_model
    seed: int = 0


class SparseDictionarySynth:
    def __init__(self, spec: SyntheticSpec, device="cpu"):
        self.spec = spec
        self.device = torch.device(device)
        g = torch.Generator(device="cpu").manual_seed(spec.seed)
        L, d, n = spec.num_layers, spec.d_model, spec.dict_size
        self.dictionary = (torch.randn(L, n, d, generator=g) / d ** 0.5).to(self.device)
        a_var = spec.a_var_scale if spec.a_var_scale is not None else 1.0 / d
        self.A: Dict[Tuple[int, int], torch.Tensor] = {}
        for l in range(L):
            for j in range(l + 1):
                self.A[(j, l)] = (torch.randn(d, d, generator=g) * (a_var / (l + 1)) ** 0.5).to(self.device)
        self.mean_in = self.std_in = self.mean_tg = self.std_tg = None

    def _gen(self, seed: int) -> torch.Generator:
        return torch.Generator(device=self.device).manual_seed(int(seed))

    @torch.no_grad()
    def sample_raw(self, n_tokens: int, seed: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Un-normalised ``(inputs, targets)`` as ``[L, n, d]`` fp32 tensors."""
        sp, dev = self.spec, self.device
        g = self._gen(seed)
        L, d, nd = sp.num_layers, sp.d_model, sp.dict_size
        max_c = int(sp.active_mean + 6 * sp.active_mean ** 0.5 + 8)
        xs = []
        for l in range(L):
            counts = torch.poisson(torch.full((n_tokens,), float(sp.active_mean), device=dev), generator=g).clamp_(max=max_c)
            idx = torch.randint(0, nd, (n_tokens, max_c), device=dev, generator=g)
            mags = -torch.log1p(-torch.rand(n_tokens, max_c, device=dev, generator=g).clamp_(max=1 - 1e-7))
            mags = mags * (torch.arange(max_c, device=dev)[None, :] < counts[:, None])
            coef = torch.zeros(n_tokens, nd, device=dev)
            coef.scatter_add_(1, idx, mags)
            x = coef @ self.dictionary[l]
            x = x + sp.input_noise * torch.randn(n_tokens, d, device=dev, generator=g)
            xs.append(x)
        ys = []
        for l in range(L):
            y = sp.output_noise * torch.randn(n_tokens, d, device=dev, generator=g)
            for j in range(l + 1):
                y = y + xs[j] @ self.A[(j, l)]
            ys.append(y)
        return torch.stack(xs), torch.stack(ys)

    @torch.no_grad()
    def fit_norm_stats(self, n_tokens: int = 8192, seed: int = 10_007) -> None:
        x, y = self.sample_raw(n_tokens, seed)
        self.mean_in, self.std_in = x.mean(dim=1), x.std(dim=1)
        self.mean_tg, self.std_tg = y.mean(dim=1), y.std(dim=1)

    @torch.no_grad()
    def sample(self, n_tokens: int, seed: int, normalize: bool = True, dtype=torch.float32):
        x, y = self.sample_raw(n_tokens, seed)
        if normalize:
            if self.mean_in is None:
                self.fit_norm_stats()
            x = (x - self.mean_in[:, None, :]) / (self.std_in[:, None, :] + 1e-6)
            y = (y - self.mean_tg[:, None, :]) / (self.std_tg[:, None, :] + 1e-6)
        return x.to(dtype), y.to(dtype)

    def norm_stats_dict(self) -> Dict[str, Dict[str, Dict[str, list]]]:
        if self.mean_in is None:
            self.fit_norm_stats()
        out = {}
        for l in range(self.spec.num_layers):
            out[str(l)] = {
                "inputs": {"mean": self.mean_in[l].tolist(), "std": self.std_in[l].tolist()},
                "targets": {"mean": self.mean_tg[l].tolist(), "std": self.std_tg[l].tolist()},
            }
        return out


def write_synthetic_dataset(
    out_dir: str,
    spec: SyntheticSpec,
    total_tokens: int,
    chunk_tokens: int,
    dtype: str = "bfloat16",
    device="cpu",
    compression: Optional[str] = None,
    model_name: str = "synthetic-sparse-dictionary",
) -> str:
    """Write a manifest dataset (HDF5 chunks + index.bin + metadata.json + norm_stats.json) of *raw*
    synthetic activations; the statistics in ``norm_stats.json`` standardise them at read time."""
    from ..io import hdf5, manifest

    os.makedirs(out_dir, exist_ok=True)
    synth = SparseDictionarySynth(spec, device=device)
    synth.fit_norm_stats()
    records = []
    written, cid, offset = 0, 0, 0
    while written < total_tokens:
        n = min(chunk_tokens, total_tokens - written)
        x, y = synth.sample_raw(n, seed=spec.seed * 1_000_003 + cid + 1)
        perm = torch.randperm(n, generator=torch.Generator().manual_seed(spec.seed + 77 * cid)).to(x.device)
        x, y = x[:, perm], y[:, perm]
        layers = {}
        for l in range(spec.num_layers):
            layers[l] = (hdf5.to_storage_array(x[l], dtype), hdf5.to_storage_array(y[l], dtype))
        hdf5.write_chunk_file(os.path.join(out_dir, f"chunk_{cid}.hdf5"), layers, compression=compression)
        records.append((cid, n, offset))
        offset += n
        written += n
        cid += 1
    manifest.write_index_3field(os.path.join(out_dir, "index.bin"), records)
    meta = {
        "model_name": model_name, "dataset": "synthetic", "split": "train", "num_layers": spec.num_layers,
        "d_model": spec.d_model, "dtype": dtype, "total_tokens": int(written), "chunk_tokens": int(chunk_tokens),
        "created": time.strftime("%Y-%m-%dT%H:%M:%S"),
    }
    with open(os.path.join(out_dir, "metadata.json"), "w") as fh:
        json.dump(meta, fh, indent=2)
    with open(os.path.join(out_dir, "norm_stats.json"), "w") as fh:
        json.dump(synth.norm_stats_dict(), fh)
    return out_dir
