"""Weights & Biases logging (reference: clt/training/wandb_logger.py:13-306).

Same key layout as the reference (``training/*`` renames, evaluation sections with histograms for
list-valued layerwise metrics, run resumption by id, artifacts).  ``wandb`` is imported lazily; when it
is missing or disabled every call is a no-op (:class:`DummyWandBLogger`).
"""
from __future__ import annotations

import dataclasses
import importlib.util
import logging
import os
import time
from typing import Any, Dict, Optional

logger = logging.getLogger(__name__)


class DummyWandBLogger:
    def __init__(self, *args, **kwargs):
        pass

    def log_step(self, *args, **kwargs):
        pass

    def log_evaluation(self, *args, **kwargs):
        pass

    def log_artifact(self, *args, **kwargs):
        pass

    def finish(self):
        pass

    def get_current_wandb_run_id(self) -> Optional[str]:
        return None


class WandBLogger:
    def __init__(self, training_config, clt_config, log_dir: str, resume_wandb_id: Optional[str] = None):
        self.enabled = bool(training_config.enable_wandb)
        self.training_config = training_config
        self.clt_config = clt_config
        self.log_dir = log_dir
        self.wandb_run = None
        self._wandb = None
        if not self.enabled:
            return
        if importlib.util.find_spec("wandb") is None:
            logger.warning("wandb is not installed; WandB logging disabled")
            self.enabled = False
            return
        import wandb

        self._wandb = wandb
        project = training_config.wandb_project or os.environ.get("WANDB_PROJECT", "crosslayer-transcoder")
        entity = training_config.wandb_entity or os.environ.get("WANDB_ENTITY")
        name = training_config.wandb_run_name or f"clt-{time.strftime('%Y%m%d-%H%M%S')}"
        cfg = {"training": dataclasses.asdict(training_config), "clt": dataclasses.asdict(clt_config)}
        kwargs: Dict[str, Any] = dict(project=project, entity=entity, name=name, config=cfg, tags=training_config.wandb_tags, dir=log_dir)
        if resume_wandb_id:
            kwargs.update(id=resume_wandb_id, resume="must")
        try:
            self.wandb_run = wandb.init(**kwargs)
        except Exception as exc:  # network / auth problems must not stop training
            logger.warning("wandb.init failed (%s); continuing without WandB", exc)
            self.enabled = False

    def get_current_wandb_run_id(self) -> Optional[str]:
        return self.wandb_run.id if self.enabled and self.wandb_run is not None else None

    def log_step(self, step: int, loss_dict: Dict[str, float], lr: Optional[float] = None,
                 sparsity_lambda: Optional[float] = None, total_tokens_processed: Optional[int] = None) -> None:
        if not self.enabled:
            return
        renames = {"total": "training/total_loss", "reconstruction": "training/reconstruction_loss",
                   "sparsity": "training/sparsity_loss", "preactivation": "training/preactivation_loss",
                   "auxiliary": "training/auxiliary_loss"}
        data = {renames.get(k, f"training/{k}"): v for k, v in loss_dict.items()}
        if lr is not None:
            data["training/learning_rate"] = lr
        if sparsity_lambda is not None:
            data["training/sparsity_lambda"] = sparsity_lambda
        if total_tokens_processed is not None:
            data["training/total_tokens_processed"] = total_tokens_processed
        self._wandb.log(data, step=step)

    def log_evaluation(self, step: int, eval_metrics: Dict[str, Any]) -> None:
        if not self.enabled:
            return
        data: Dict[str, Any] = {}
        for key, value in eval_metrics.items():
            if isinstance(value, dict):  # layerwise/<metric> -> {layer_i: scalar | list}
                for layer, v in value.items():
                    if isinstance(v, (list, tuple)):
                        if len(v):
                            data[f"{key}/{layer}"] = self._wandb.Histogram(v)
                    else:
                        data[f"{key}/{layer}"] = v
            elif isinstance(value, (list, tuple)):
                if len(value):
                    data[key] = self._wandb.Histogram(value)
            else:
                data[key] = value
        self._wandb.log(data, step=step)

    def log_artifact(self, artifact_path: str, artifact_type: str, name: Optional[str] = None) -> None:
        if not self.enabled or not os.path.exists(artifact_path):
            return
        art = self._wandb.Artifact(name or os.path.basename(artifact_path), type=artifact_type)
        if os.path.isdir(artifact_path):
            art.add_dir(artifact_path)
        else:
            art.add_file(artifact_path)
        self.wandb_run.log_artifact(art)

    def finish(self) -> None:
        if self.enabled and self.wandb_run is not None:
            self.wandb_run.finish()
