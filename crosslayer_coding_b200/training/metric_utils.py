"""Step-metric bookkeeping (reference: clt/training/metric_utils.py:16-88).

Keeps ``{"train_losses": [...], "eval_metrics": [...]}`` and writes ``metrics.json`` into the run
directory every ``log_interval`` steps and after every evaluation.  Unlike the reference, training
losses may be handed over as device scalars: they are kept on the device and read back in one
transfer when the file is written, so logging does not add a host sync to every step.
"""
from __future__ import annotations

import json
import logging
import os
import time
from typing import Any, Dict, List, Optional

import torch

logger = logging.getLogger(__name__)

LOSS_KEYS = ("total", "reconstruction", "sparsity", "preactivation", "auxiliary")


class MetricLogger:
    def __init__(self, distributed: bool, rank: int, log_dir: str, wandb_logger, training_config, world_size: int = 1):
        self.distributed = distributed
        self.rank = rank
        self.log_dir = log_dir
        self.wandb_logger = wandb_logger
        self.training_config = training_config
        self.world_size = world_size
        self.metrics: Dict[str, List[Dict[str, Any]]] = {"train_losses": [], "eval_metrics": []}
        self._pending: List[Any] = []  # (step, stacked device tensor, lr, lambda)

    def _flush_pending(self) -> None:
        if not self._pending:
            return
        stacked = torch.stack([p[1] for p in self._pending]).float().cpu().tolist()
        for (step, _, lr, lam), vals in zip(self._pending, stacked):
            entry = {"step": step, **dict(zip(LOSS_KEYS, vals))}
            self.metrics["train_losses"].append(entry)
            if self.wandb_logger is not None and (not self.distributed or self.rank == 0):
                tokens = self.training_config.train_batch_size_tokens * (step + 1)
                self.wandb_logger.log_step(step, dict(zip(LOSS_KEYS, vals)), lr=lr, sparsity_lambda=lam, total_tokens_processed=tokens)
        self._pending.clear()

    def log_training_step(
        self,
        step: int,
        loss_dict: Dict[str, Any],
        current_lr: Optional[float] = None,
        current_sparsity_lambda: Optional[float] = None,
    ) -> None:
        if isinstance(loss_dict.get("_vector"), torch.Tensor):
            # the fused step hands over its loss terms as one device vector in LOSS_KEYS order: nothing to launch here
            self._pending.append((step, loss_dict["_vector"][: len(LOSS_KEYS)], current_lr, current_sparsity_lambda))
        elif any(isinstance(v, torch.Tensor) for v in loss_dict.values()):
            dev = next(v.device for v in loss_dict.values() if isinstance(v, torch.Tensor))
            vec = torch.stack([
                (loss_dict.get(k) if isinstance(loss_dict.get(k), torch.Tensor) else torch.tensor(float(loss_dict.get(k, 0.0)), device=dev)).detach().float().reshape(())
                for k in LOSS_KEYS
            ])
            self._pending.append((step, vec, current_lr, current_sparsity_lambda))
        else:
            self.metrics["train_losses"].append({"step": step, **{k: float(v) for k, v in loss_dict.items() if not k.startswith("_")}})
            if self.wandb_logger is not None and (not self.distributed or self.rank == 0):
                tokens = self.training_config.train_batch_size_tokens * (step + 1)
                self.wandb_logger.log_step(step, loss_dict, lr=current_lr, sparsity_lambda=current_sparsity_lambda,
                                           total_tokens_processed=tokens)
        interval = max(1, self.training_config.log_interval)
        if step % interval == 0:
            self._save_metrics_to_disk()

    def log_evaluation_metrics(self, step: int, eval_metrics_dict: Dict[str, Any]) -> None:
        if not self.distributed or self.rank == 0:
            self.metrics["eval_metrics"].append({"step": step, **eval_metrics_dict})
            if self.wandb_logger is not None:
                self.wandb_logger.log_evaluation(step, eval_metrics_dict)
            self._save_metrics_to_disk()

    def _save_metrics_to_disk(self) -> None:
        self._flush_pending()
        if self.distributed and self.rank != 0:
            return
        path = os.path.join(self.log_dir, "metrics.json")
        tmp = path + ".tmp"
        try:
            with open(tmp, "w") as fh:
                json.dump(self.metrics, fh, indent=2, default=lambda o: float(o) if hasattr(o, "__float__") else str(o))
            os.replace(tmp, path)
        except OSError as exc:
            logger.warning("Rank %d: failed to save metrics to %s: %s", self.rank, path, exc)
