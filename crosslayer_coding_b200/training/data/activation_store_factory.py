"""Build the activation store named by ``TrainingConfig.activation_source``
(reference: clt/training/data/activation_store_factory.py:12-102)."""
from __future__ import annotations

import logging
from typing import Any

import torch

from ...config import CLTConfig, TrainingConfig
from .base_store import BaseActivationStore

logger = logging.getLogger(__name__)


def create_activation_store(
    training_config: TrainingConfig,
    clt_config: CLTConfig,
    device: Any,
    rank: int = 0,
    world: int = 1,
    start_time: float = 0.0,
    shard_data: bool = True,
    shard_group=None,
) -> BaseActivationStore:
    tc = training_config
    common = dict(
        train_batch_size_tokens=tc.train_batch_size_tokens, device=torch.device(device), dtype=tc.activation_dtype,
        rank=rank, world=world, seed=tc.seed, sampling_strategy=tc.sampling_strategy,
        normalization_method=tc.normalization_method, shard_data=shard_data,
        prefetch_batches=tc.prefetch_batches, auto_advance_epoch=tc.auto_advance_epoch,
    )
    if tc.activation_source == "local_manifest":
        if not tc.activation_path:
            raise ValueError("activation_path must be set in TrainingConfig when activation_source is 'local_manifest'.")
        from .local_activation_store import LocalActivationStore

        # tensor-parallel runs on GPUs: every rank assembles and copies 1/W of each batch, the rest arrives over NVLink
        store: BaseActivationStore = LocalActivationStore(dataset_path=tc.activation_path, shard_group=shard_group, **common)
    elif tc.activation_source == "remote":
        rc = tc.remote_config or {}
        if not rc.get("server_url") or not rc.get("dataset_id"):
            raise ValueError("remote_config needs 'server_url' and 'dataset_id'")
        from .remote_activation_store import RemoteActivationStore

        if "prefetch_batches" in rc:
            common["prefetch_batches"] = int(rc["prefetch_batches"])
        store = RemoteActivationStore(
            server_url=rc["server_url"], dataset_id=rc["dataset_id"], timeout=rc.get("timeout", 60),
            max_retries=rc.get("max_retries", 3), **common,
        )
    else:
        raise ValueError(f"Unknown activation_source: {tc.activation_source}. Valid options: 'local_manifest', 'remote'.")
    if hasattr(store, "d_model") and store.d_model != clt_config.d_model:
        logger.warning("store d_model %d differs from CLT d_model %d", store.d_model, clt_config.d_model)
    if hasattr(store, "num_layers") and store.num_layers != clt_config.num_layers:
        logger.warning("store has %d layers, CLT has %d", store.num_layers, clt_config.num_layers)
    return store
