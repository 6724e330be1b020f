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
* files are written to a temporary name and renamed, so an interrupted save never leaves a torn file;
* every file is written once: the ``latest`` copies are hard links of the step files (a copy only where the
  file system has no hard links);
* with ``async_save`` the tensors are copied device -> pinned host on a side stream and the files are written
  by a background thread, so the step loop only waits for the copy engine (``wait()`` joins the writer; it is
  called before the next save, before a load and when training ends).
"""
from __future__ import annotations

import json
import logging
import os
import shutil
import threading
import time
from typing import Any, Callable, Dict, List, Optional

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


def _link_or_copy(src: str, dst: str) -> None:
    """``dst`` becomes a second name of ``src`` (hard link, atomic replace); a copy where links are unsupported."""
    tmp = dst + ".tmp"
    if os.path.lexists(tmp):
        os.remove(tmp)
    try:
        os.link(src, tmp)
    except OSError:
        shutil.copy2(src, tmp)
    os.replace(tmp, dst)


def snapshot_to_host(tensors: Dict[str, torch.Tensor], stream=None) -> Dict[str, torch.Tensor]:
    """Host copies of ``tensors`` that no longer alias the live parameters.  CUDA tensors are copied into pinned
    memory with non-blocking copies on ``stream`` (ordered after the work queued so far on the current stream);
    the caller synchronises the returned event-less copies with ``stream.synchronize()`` before reading them."""
    out: Dict[str, torch.Tensor] = {}
    cuda = [v for v in tensors.values() if v.is_cuda]
    if cuda and stream is not None:
        stream.wait_stream(torch.cuda.current_stream(cuda[0].device))
        with torch.cuda.stream(stream):
            for k, v in tensors.items():
                if v.is_cuda:
                    src = v.detach().contiguous()
                    src.record_stream(stream)
                    host = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
                    host.copy_(src, non_blocking=True)
                    out[k] = host
                else:
                    out[k] = v.detach().clone().contiguous()
        return out
    for k, v in tensors.items():
        out[k] = (v.detach().cpu() if v.is_cuda else v.detach().clone()).contiguous()
    return out


def _wait_for_files(paths: List[str], timeout_s: float) -> bool:
    """True once every path exists (files appear by atomic rename, so existence means complete)."""
    deadline = time.monotonic() + timeout_s
    while True:
        if all(os.path.exists(p) for p in paths):
            return True
        if time.monotonic() > deadline:
            return False
        time.sleep(0.02)


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
    from ..models.base import shard_width

    local = shard_width(num_features, world)
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


def optimizer_shard_axis(name: str, tensor: torch.Tensor) -> Optional[int]:
    """Feature axis of an optimizer tensor (fused-engine names and ``param::field`` names of the autograd
    optimizer), or None for replicated / scalar state."""
    if tensor.dim() == 0:
        return None
    base = name.split("::", 1)[0]
    if name.endswith("::step"):
        return None
    if base in ("enc_m", "enc_v", "encb_m", "encb_v", "theta_m", "theta_v", "enc_weight", "enc_bias", "log_threshold",
                "feature_offset", "feature_scale", "dead_counter_2d", "foff_m", "foff_v", "fsc_m", "fsc_v"):
        return 1
    if base.startswith(("dec_m.", "dec_v.", "dec_weight.")):
        return 0
    return None  # decoder biases, skip weights, step counters


def reshard_optimizer_tensors(per_rank: List[Dict[str, torch.Tensor]], num_features: int, num_layers: int,
                              new_rank: int, new_world: int) -> Dict[str, torch.Tensor]:
    """Optimizer state saved by ``len(per_rank)`` ranks, re-cut for rank ``new_rank`` of ``new_world``: sharded
    moments are concatenated along their feature axis, the padding is dropped and the new shard is sliced out
    (zero-padded to the new shard width); replicated tensors come from rank 0.  The fused engine's flat
    ``dead_counter`` ``[L * F_local]`` is handled as ``[L, F_local]``."""
    from ..models.base import shard_width

    new_local = shard_width(num_features, new_world)
    start = new_rank * new_local
    valid = max(0, min(num_features, start + new_local) - start)
    out: Dict[str, torch.Tensor] = {}
    for name, t0 in per_rank[0].items():
        flat_counter = name == "dead_counter" and t0.dim() == 1
        parts = [r[name] for r in per_rank]
        if flat_counter:
            parts = [p.view(num_layers, -1) for p in parts]
            axis: Optional[int] = 1
        else:
            axis = optimizer_shard_axis(name, t0)
        if axis is None:
            out[name] = t0
            continue
        full = torch.cat(parts, dim=axis).narrow(axis, 0, num_features)
        piece = full.narrow(axis, start, valid) if valid > 0 else full.narrow(axis, 0, 0)
        if valid < new_local:
            pad_shape = list(full.shape)
            pad_shape[axis] = new_local - valid
            piece = torch.cat([piece, torch.zeros(pad_shape, dtype=full.dtype)], dim=axis)
        piece = piece.contiguous()
        out[name] = piece.reshape(-1) if flat_counter else piece
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
        async_save: bool = False,
        merge_timeout_s: float = 600.0,
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
        self.async_save = bool(async_save)
        self.merge_timeout_s = float(merge_timeout_s)
        self._writer: Optional[threading.Thread] = None
        self._writer_error: Optional[BaseException] = None
        self._copy_stream = None

    # --------------------------------------------------------------------- save
    def _save_checkpoint(self, step: int, trainer_state_to_save: Dict[str, Any], optimizer_tensors: Optional[Dict[str, torch.Tensor]] = None) -> None:
        """``optimizer_tensors``: this rank's optimizer moments as a flat ``{name: tensor}`` mapping (saved
        as safetensors next to the weights); everything picklable goes into ``trainer_state_to_save``."""
        try:
            self.wait()  # one save in flight at a time
            if self.distributed:
                self._save_distributed(step, trainer_state_to_save, optimizer_tensors)
            else:
                self._save_single(step, trainer_state_to_save, optimizer_tensors)
        except (OSError, SafetensorError) as exc:  # checkpoint IO problems are logged, not fatal (reference behaviour)
            logger.warning("Rank %d: failed to save checkpoint at step %d: %s", self.rank, step, exc)

    def wait(self) -> None:
        """Join the background writer of the last asynchronous save (no-op otherwise)."""
        w = self._writer
        if w is not None:
            w.join()
            self._writer = None
        if self._writer_error is not None:
            exc, self._writer_error = self._writer_error, None
            logger.warning("Rank %d: background checkpoint write failed: %s", self.rank, exc)

    def _store_state(self):
        return self.activation_store.state_dict() if self.activation_store is not None else None

    def _snapshot(self, tensors: Optional[Dict[str, torch.Tensor]]):
        """Host copy of ``tensors`` and a callable that makes the copy readable (waits for the copy stream)."""
        if not tensors:
            return {}, (lambda: None)
        use_stream = self.async_save and torch.cuda.is_available() and any(v.is_cuda for v in tensors.values())
        if use_stream:
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream(device=self.device)
            host = snapshot_to_host(tensors, self._copy_stream)
            ev = torch.cuda.Event()
            ev.record(self._copy_stream)
            # the step loop may overwrite the parameters only after the copy has read them
            torch.cuda.current_stream(self.device).wait_event(ev)
            return host, ev.synchronize
        return snapshot_to_host(tensors, None), (lambda: None)

    def _run(self, job: Callable[[], None]) -> None:
        if not self.async_save:
            job()
            return

        def guarded():
            try:
                job()
            except BaseException as exc:  # noqa: BLE001 - reported by wait()
                self._writer_error = exc

        self._writer = threading.Thread(target=guarded, name="clt-checkpoint-writer", daemon=False)
        self._writer.start()

    def _save_single(self, step, trainer_state, optimizer_tensors) -> None:
        os.makedirs(self.log_dir, exist_ok=True)
        sd, sd_ready = self._snapshot(self.model.state_dict())
        opt, opt_ready = self._snapshot(optimizer_tensors)
        store_state = self._store_state()
        d = self.log_dir

        def write():
            sd_ready()
            opt_ready()
            files = [(f"clt_checkpoint_{step}.safetensors", f"clt_checkpoint_latest.safetensors", lambda p: _atomic_save_safetensors(sd, p))]
            if store_state is not None:
                files.append((f"activation_store_{step}.pt", "activation_store_latest.pt", lambda p: _atomic_torch_save(store_state, p)))
            files.append((f"trainer_state_{step}.pt", "trainer_state_latest.pt", lambda p: _atomic_torch_save(trainer_state, p)))
            if opt:
                files.append((f"optimizer_{step}.safetensors", "optimizer_latest.safetensors", lambda p: _atomic_save_safetensors(opt, p)))
            for name, latest, writer in files:
                writer(os.path.join(d, name))
                _link_or_copy(os.path.join(d, name), os.path.join(d, latest))
            if self.wandb_logger is not None:
                self.wandb_logger.log_artifact(os.path.join(d, f"clt_checkpoint_{step}.safetensors"), "model", f"clt_checkpoint_{step}")

        self._run(write)

    def _shard_meta(self) -> Dict[str, Any]:
        m = self.model
        return {
            "world_size": self.world_size,
            "num_features": m.config.num_features,
            "num_layers": m.config.num_layers,
            "local_features": m.local_features,
            "dtype": str(m.dtype).replace("torch.", ""),
            "format": "crosslayer_coding_b200.sharded.v1",
        }

    def _save_distributed(self, step, trainer_state, optimizer_tensors) -> None:
        step_dir = os.path.join(self.log_dir, f"step_{step}")
        latest_dir = os.path.join(self.log_dir, "latest")
        os.makedirs(step_dir, exist_ok=True)
        # a stale shard of the same step (an earlier run into this directory) would satisfy rank 0's wait-for-files:
        # every rank removes its own before the barrier
        for name in (f"rank_{self.rank}_model.safetensors", f"rank_{self.rank}_optim.safetensors"):
            if os.path.exists(os.path.join(step_dir, name)):
                os.remove(os.path.join(step_dir, name))
        self._barrier()
        sd, sd_ready = self._snapshot(self.model.state_dict())
        opt, opt_ready = self._snapshot(optimizer_tensors)
        store_state = self._store_state() if self.rank == 0 else None
        meta = self._shard_meta()
        rank, world, F = self.rank, self.world_size, self.model.config.num_features

        def write():
            sd_ready()
            opt_ready()
            if opt:  # the model shard is written last: its presence tells rank 0 that this rank is complete
                _atomic_save_safetensors(opt, os.path.join(step_dir, f"rank_{rank}_optim.safetensors"))
            _atomic_save_safetensors(sd, os.path.join(step_dir, f"rank_{rank}_model.safetensors"))
            if rank != 0:
                return
            shard_files = [os.path.join(step_dir, f"rank_{r}_model.safetensors") for r in range(world)]
            if not _wait_for_files(shard_files, self.merge_timeout_s):
                raise OSError(f"checkpoint step {step}: not every rank's shard appeared within {self.merge_timeout_s:.0f} s")
            merged = merge_shards([load_safetensors_file(p) for p in shard_files], F)
            _atomic_save_safetensors(merged, os.path.join(step_dir, "model.safetensors"))
            if store_state is not None:
                _atomic_torch_save(store_state, os.path.join(step_dir, "activation_store.pt"))
            _atomic_torch_save(trainer_state, os.path.join(step_dir, "trainer_state.pt"))
            with open(os.path.join(step_dir, "shard_meta.json"), "w") as fh:
                json.dump(meta, fh, indent=2)
            tmp_latest = latest_dir + ".tmp"
            if os.path.isdir(tmp_latest):
                shutil.rmtree(tmp_latest)
            os.makedirs(tmp_latest)
            for name in os.listdir(step_dir):
                if not name.endswith(".tmp"):
                    _link_or_copy(os.path.join(step_dir, name), os.path.join(tmp_latest, name))
            if os.path.isdir(latest_dir):
                shutil.rmtree(latest_dir)
            os.replace(tmp_latest, latest_dir)
            self._prune_old()
            if self.wandb_logger is not None:
                self.wandb_logger.log_artifact(step_dir, "model", f"dist_checkpoint_{step}")

        self._run(write)
        if not self.async_save:
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
        self.wait()
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
                meta = json.load(fh)
            saved_world = int(meta.get("world_size", 0)) or None
            if saved_world == self.world_size and int(meta.get("local_features", self.model.local_features)) != self.model.local_features:
                saved_world = -saved_world  # same world size, other shard width: go through the merged model
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
            # other world size (or shard width): re-cut the moments, counters and thresholds' state for this rank
            paths = [os.path.join(ckpt_dir, f"rank_{r}_optim.safetensors") for r in range(abs(saved_world))]
            if all(os.path.exists(p) for p in paths):
                state["optimizer_tensors"] = reshard_optimizer_tensors(
                    [load_safetensors_file(p) for p in paths], F, self.model.config.num_layers, self.rank, self.world_size)
                state["optimizer_resharded_from"] = abs(saved_world)
            else:
                logger.warning("Rank %d: %s holds no complete set of optimizer shards; the optimizer state starts fresh", self.rank, ckpt_dir)
        return state
