"""Checkpoint save / load with sharded safetensors (reference: clt/training/checkpointing.py:27-533).

File layout kept from the reference:

* single process: ``clt_checkpoint_{step}.safetensors`` + ``clt_checkpoint_latest.safetensors`` (full
  ``state_dict`` under the reference key names), ``activation_store_{step|latest}.pt``,
  ``trainer_state_{step|latest}.pt``;
* distributed: directories ``step_{N}/`` and ``latest/`` with a merged ``model.safetensors`` (encoder
  weights concatenated on dim 0, decoder weights on dim 1), ``activation_store.pt``, ``trainer_state.pt``;
  only the newest three ``step_*`` directories are kept.

Differences (the reference's distributed load path cannot work, see checkpointing.py:309-337):

* every rank writes ``rank_{r}_model.safetensors`` *and* ``rank_{r}_optim.safetensors`` (the reference
  pickles the model shard and saves rank 0's optimizer state only);
* ``shard_meta.json`` records world size, padded shard width and dtype, so a checkpoint can be loaded at a
  different world size (re-sharded from the merged model; optimizer moments are re-sharded too);
* feature-sharded tensors (``log_threshold``, ``feature_offset``, ``feature_scale``) are merged along the
  feature axis (the reference concatenates the replicated ``log_threshold`` to ``[L, F*W]`` and keeps rank
  0's affine shard);
* files are written to a temporary name and renamed, so an interrupted save never leaves a torn file.
"""
from __future__ import annotations

import json
import logging
import os
import shutil
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
from safetensors.torch import load_file as load_safetensors_file
from safetensors.torch import save_file as save_safetensors_file

try:
    from safetensors import SafetensorError
except ImportError:  # very old safetensors
    SafetensorError = OSError  # type: ignore[misc,assignment]

logger = logging.getLogger(__name__)

_FEATURE_DIM0 = ("encoder_module.encoders.",)  # weight [F_local, d], bias_param [F_local]
_FEATURE_LAST = ("decoder_module.feature_offset.", "decoder_module.feature_scale.")


def _atomic_save_safetensors(tensors: Dict[str, torch.Tensor], path: str) -> None:
    tmp = path + ".tmp"
    # every tensor gets its own host storage: state-dict entries are views of the packed parameters
    host = {k: (v.detach().cpu() if v.is_cuda else v.detach().clone()).contiguous() for k, v in tensors.items()}
    save_safetensors_file(host, tmp)
    os.replace(tmp, path)


def _atomic_torch_save(obj: Any, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def shard_axis(key: str, tensor: torch.Tensor) -> Optional[int]:
    """Axis along which a reference-named tensor is sharded over the feature dimension, or None."""
    if key.startswith("encoder_module.encoders."):
        return 0
    if key.startswith("decoder_module.decoders.") and key.endswith(".weight"):
        return 1
    if key.startswith(_FEATURE_LAST):
        return 0
    if key == "theta_manager.log_threshold":
        return 1
    return None


def merge_shards(shards: List[Dict[str, torch.Tensor]], num_features: int) -> Dict[str, torch.Tensor]:
    """Concatenate per-rank state dicts (reference key names) into the full model and drop padding."""
    out: Dict[str, torch.Tensor] = {}
    for key, t0 in shards[0].items():
        axis = shard_axis(key, t0)
        if axis is None or len(shards) == 1:
            out[key] = t0
            continue
        full = torch.cat([s[key] for s in shards], dim=axis)
        out[key] = full.narrow(axis, 0, num_features).contiguous()
    return out


def slice_for_rank(full: Dict[str, torch.Tensor], rank: int, world: int, num_features: int) -> Dict[str, torch.Tensor]:
    """Inverse of :func:`merge_shards`: this rank's (zero-padded) shard of a full state dict."""
    local = -(-num_features // world)
    start = rank * local
    out: Dict[str, torch.Tensor] = {}
    for key, t in full.items():
        axis = shard_axis(key, t)
        if axis is None or world == 1:
            out[key] = t
            continue
        valid = max(0, min(num_features, start + local) - start)
        piece = t.narrow(axis, start, valid) if valid > 0 else t.narrow(axis, 0, 0)
        if valid < local:
            pad_shape = list(t.shape)
            pad_shape[axis] = local - valid
            fill = 0.0
            piece = torch.cat([piece, torch.full(pad_shape, fill, dtype=t.dtype)], dim=axis)
        out[key] = piece.contiguous()
    return out


class CheckpointManager:
    def __init__(
        self,
        model,
        activation_store,
        wandb_logger,
        log_dir: str,
        distributed: bool,
        rank: int,
        device: torch.device,
        world_size: int = 1,
        keep_n_checkpoints: int = 3,
    ):
        self.model = model
        self.activation_store = activation_store
        self.wandb_logger = wandb_logger
        self.log_dir = log_dir
        self.distributed = distributed
        self.rank = rank
        self.device = device
        self.world_size = world_size
        self.keep_n_checkpoints = keep_n_checkpoints

    # --------------------------------------------------------------------- save
    def _save_checkpoint(self, step: int, trainer_state_to_save: Dict[str, Any], optimizer_tensors: Optional[Dict[str, torch.Tensor]] = None) -> None:
        """``optimizer_tensors``: this rank's optimizer moments as a flat ``{name: tensor}`` mapping (saved
        as safetensors next to the weights); everything picklable goes into ``trainer_state_to_save``."""
        try:
            if self.distributed:
                self._save_distributed(step, trainer_state_to_save, optimizer_tensors)
            else:
                self._save_single(step, trainer_state_to_save, optimizer_tensors)
        except (OSError, SafetensorError) as exc:  # checkpoint IO problems are logged, not fatal (reference behaviour)
            logger.warning("Rank %d: failed to save checkpoint at step %d: %s", self.rank, step, exc)

    def _store_state(self):
        return self.activation_store.state_dict() if self.activation_store is not None else None

    def _save_single(self, step, trainer_state, optimizer_tensors) -> None:
        os.makedirs(self.log_dir, exist_ok=True)
        sd = self.model.state_dict()
        for tag in (str(step), "latest"):
            _atomic_save_safetensors(sd, os.path.join(self.log_dir, f"clt_checkpoint_{tag}.safetensors"))
            store_state = self._store_state()
            if store_state is not None:
                _atomic_torch_save(store_state, os.path.join(self.log_dir, f"activation_store_{tag}.pt"))
            _atomic_torch_save(trainer_state, os.path.join(self.log_dir, f"trainer_state_{tag}.pt"))
            if optimizer_tensors:
                _atomic_save_safetensors(optimizer_tensors, os.path.join(self.log_dir, f"optimizer_{tag}.safetensors"))
        if self.wandb_logger is not None:
            self.wandb_logger.log_artifact(os.path.join(self.log_dir, f"clt_checkpoint_{step}.safetensors"), "model", f"clt_checkpoint_{step}")

    def _shard_meta(self) -> Dict[str, Any]:
        m = self.model
        return {
            "world_size": self.world_size,
            "num_features": m.config.num_features,
            "local_features": m.local_features,
            "dtype": str(m.dtype).replace("torch.", ""),
            "format": "crosslayer_coding_b200.sharded.v1",
        }

    def _save_distributed(self, step, trainer_state, optimizer_tensors) -> None:
        step_dir = os.path.join(self.log_dir, f"step_{step}")
        latest_dir = os.path.join(self.log_dir, "latest")
        os.makedirs(step_dir, exist_ok=True)
        self._barrier()
        sd = self.model.state_dict()
        _atomic_save_safetensors(sd, os.path.join(step_dir, f"rank_{self.rank}_model.safetensors"))
        if optimizer_tensors:
            _atomic_save_safetensors(optimizer_tensors, os.path.join(step_dir, f"rank_{self.rank}_optim.safetensors"))
        self._barrier()
        if self.rank == 0:
            shards = [load_safetensors_file(os.path.join(step_dir, f"rank_{r}_model.safetensors")) for r in range(self.world_size)]
            merged = merge_shards(shards, self.model.config.num_features)
            _atomic_save_safetensors(merged, os.path.join(step_dir, "model.safetensors"))
            store_state = self._store_state()
            if store_state is not None:
                _atomic_torch_save(store_state, os.path.join(step_dir, "activation_store.pt"))
            _atomic_torch_save(trainer_state, os.path.join(step_dir, "trainer_state.pt"))
            with open(os.path.join(step_dir, "shard_meta.json"), "w") as fh:
                json.dump(self._shard_meta(), fh, indent=2)
            tmp_latest = latest_dir + ".tmp"
            if os.path.isdir(tmp_latest):
                shutil.rmtree(tmp_latest)
            shutil.copytree(step_dir, tmp_latest)
            if os.path.isdir(latest_dir):
                shutil.rmtree(latest_dir)
            os.replace(tmp_latest, latest_dir)
            self._prune_old()
            if self.wandb_logger is not None:
                self.wandb_logger.log_artifact(step_dir, "model", f"dist_checkpoint_{step}")
        self._barrier()

    def _prune_old(self) -> None:
        dirs = []
        for name in os.listdir(self.log_dir):
            if name.startswith("step_") and os.path.isdir(os.path.join(self.log_dir, name)):
                try:
                    dirs.append((int(name.split("_", 1)[1]), name))
                except ValueError:
                    continue
        for _, name in sorted(dirs)[: -self.keep_n_checkpoints]:
            shutil.rmtree(os.path.join(self.log_dir, name), ignore_errors=True)

    def _barrier(self) -> None:
        if self.distributed and dist.is_available() and dist.is_initialized():
            dist.barrier()

    # --------------------------------------------------------------------- load
    def load_checkpoint(self, checkpoint_path: str) -> Dict[str, Any]:
        """Load model (+ activation store) from ``checkpoint_path`` (a ``.safetensors`` file or a
        ``step_N`` / ``latest`` directory) and return the trainer state dict; optimizer tensors, when
        present, come back under ``"optimizer_tensors"``."""
        if os.path.isdir(checkpoint_path):
            return self._load_dir(checkpoint_path)
        return self._load_file(checkpoint_path)

    def _load_file(self, path: str) -> Dict[str, Any]:
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        full = load_safetensors_file(path)
        self.model.load_state_dict(slice_for_rank(full, self.rank, self.world_size, self.model.config.num_features)
                                   if self.world_size > 1 else full)
        base, name = os.path.dirname(path), os.path.basename(path)
        tag = name.replace("clt_checkpoint_", "").replace(".safetensors", "")
        state: Dict[str, Any] = {}
        ts = os.path.join(base, f"trainer_state_{tag}.pt")
        if os.path.exists(ts):
            state = torch.load(ts, map_location="cpu", weights_only=False)
        st = os.path.join(base, f"activation_store_{tag}.pt")
        if os.path.exists(st) and self.activation_store is not None:
            self.activation_store.load_state_dict(torch.load(st, map_location="cpu", weights_only=False))
        opt = os.path.join(base, f"optimizer_{tag}.safetensors")
        if os.path.exists(opt):
            state["optimizer_tensors"] = load_safetensors_file(opt)
        return state

    def _load_dir(self, ckpt_dir: str) -> Dict[str, Any]:
        meta_path = os.path.join(ckpt_dir, "shard_meta.json")
        saved_world = None
        if os.path.exists(meta_path):
            with open(meta_path) as fh:
                saved_world = int(json.load(fh).get("world_size", 0)) or None
        F = self.model.config.num_features
        own = os.path.join(ckpt_dir, f"rank_{self.rank}_model.safetensors")
        if saved_world == self.world_size and os.path.exists(own):
            self.model.load_state_dict(load_safetensors_file(own))
        else:
            merged = os.path.join(ckpt_dir, "model.safetensors")
            if not os.path.exists(merged):
                raise FileNotFoundError(f"no shard for rank {self.rank} and no merged model in {ckpt_dir}")
            full = load_safetensors_file(merged)
            self.model.load_state_dict(slice_for_rank(full, self.rank, self.world_size, F))
        state: Dict[str, Any] = {}
        ts = os.path.join(ckpt_dir, "trainer_state.pt")
        if os.path.exists(ts):
            state = torch.load(ts, map_location="cpu", weights_only=False)
        st = os.path.join(ckpt_dir, "activation_store.pt")
        if os.path.exists(st) and self.activation_store is not None:
            self.activation_store.load_state_dict(torch.load(st, map_location="cpu", weights_only=False))
        opt_own = os.path.join(ckpt_dir, f"rank_{self.rank}_optim.safetensors")
        if saved_world == self.world_size and os.path.exists(opt_own):
            state["optimizer_tensors"] = load_safetensors_file(opt_own)
        elif saved_world is not None:
            paths = [os.path.join(ckpt_dir, f"rank_{r}_optim.safetensors") for r in range(saved_world)]
            if all(os.path.exists(p) for p in paths):
                state["optimizer_tensors_all_ranks"] = [load_safetensors_file(p) for p in paths]
                state["optimizer_saved_world"] = saved_world
        return state
