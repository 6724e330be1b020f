"""Helpers shared by the tutorial scripts: a small synthetic dataset and tiny model/training settings, so that
every walk-through runs in a minute on a CPU (and unchanged, faster, on a B200)."""
from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO))

from crosslayer_coding_b200 import CLTConfig, TrainingConfig  # noqa: E402
from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset  # noqa: E402

L, D, DICT = 4, 64, 256


def workdir(name: str) -> str:
    root = os.environ.get("CLT_TUTORIAL_DIR", os.path.join(tempfile.gettempdir(), "clt_tutorials"))
    path = os.path.join(root, name)
    os.makedirs(path, exist_ok=True)
    return path


def dataset(path: str, tokens: int = 8192, dtype: str = "float32") -> str:
    """Write (once) a synthetic activation dataset in the on-disk layout every store reads:
    ``chunk_*.hdf5`` + ``index.bin`` + ``metadata.json`` + ``norm_stats.json``."""
    if not os.path.exists(os.path.join(path, "metadata.json")):
        spec = SyntheticSpec(num_layers=L, d_model=D, dict_size=DICT, active_mean=8, seed=0)
        write_synthetic_dataset(path, spec, total_tokens=tokens, chunk_tokens=2048, dtype=dtype, device="cpu")
    return path


def device() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def clt_config(**kw) -> CLTConfig:
    base = dict(num_features=512, num_layers=L, d_model=D, activation_fn="batchtopk", batchtopk_k=16, model_name="synthetic")
    base.update(kw)
    return CLTConfig(**base)


def training_config(data: str, steps: int = 60, **kw) -> TrainingConfig:
    base = dict(learning_rate=3e-3, training_steps=steps, train_batch_size_tokens=256, activation_source="local_manifest",
                activation_path=data, activation_dtype="float32", normalization_method="auto", sparsity_lambda=0.0,
                preactivation_coef=0.0, apply_sparsity_penalty_to_batchtopk=False, log_interval=20, eval_interval=30,
                checkpoint_interval=30, lr_scheduler="linear_final20")
    base.update(kw)
    return TrainingConfig(**base)
