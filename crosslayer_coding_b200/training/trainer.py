"""Training runtime (reference: clt/training/trainer.py:39-1121).

``CLTTrainer(clt_config, training_config, log_dir, device, distributed, resume_from_checkpoint_path).train()``
keeps the reference's contract: one process per GPU under ``torchrun`` (NCCL on GPUs, Gloo on CPU), features
tensor-parallel over the world group, every rank consuming the same batch, checkpoints / ``metrics.json`` /
``cfg.json`` in the run directory, evaluation and checkpoint cadence from the config.

The step itself has two implementations behind one interface:

* **fused** (``training/fused_engine.py``): the sm_100a kernel sequence, used whenever the configuration is
  covered (BatchTopK, bf16 weights); nothing in it synchronises with the host — losses stay on the device and
  are read back when metrics are written;
* **autograd**: the PyTorch path (any activation, tying, dtype, CPU/Gloo), with one encoder pass per step
  (the reference runs two to four, trainer.py:668 + losses.py:357,248,285).

Other deliberate differences from the reference: the learning-rate schedule is evaluated in closed form per
step (same curves as LinearLR / CosineAnnealingLR / the "linear_final20" lambda); dead-feature counters live
with the feature shard (no all-reduce(MIN) of an ``[L, F]`` int64 tensor every step, trainer.py:802); the
activation store wraps around to a new epoch instead of ending training when one pass is exhausted.
"""
from __future__ import annotations

import dataclasses
import json
import logging
import math
import os
import random
import time
from typing import Any, Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..config import CLTConfig, TrainingConfig
from ..models import CrossLayerTranscoder
from ..parallel import ops as pops
from .checkpointing import CheckpointManager
from .data.base_store import BaseActivationStore, LayerBatch
from .evaluator import CLTEvaluator
from .losses import LossManager, sparsity_lambda_at
from .metric_utils import MetricLogger
from .profiler import CUDAMemoryProfiler, DistributedProfiler, TrainingProfiler
from .wandb_logger import DummyWandBLogger, WandBLogger

logger = logging.getLogger(__name__)


def learning_rate_at(tc: TrainingConfig, step: int) -> float:
    """Learning rate used for optimisation step ``step`` (0-based)."""
    base, T = tc.learning_rate, tc.training_steps
    params = tc.lr_scheduler_params or {}
    kind = tc.lr_scheduler
    if kind is None:
        return base
    if kind == "linear":
        start, end = params.get("start_factor", 1.0), params.get("end_factor", 0.1)
        frac = min(step, T) / T
        return base * (start + (end - start) * frac)
    if kind == "cosine":
        eta_min = params.get("eta_min", 0.0)
        t_max = params.get("T_max", T)
        return eta_min + (base - eta_min) * (1 + math.cos(math.pi * step / t_max)) / 2
    if kind == "linear_final20":
        frac = params.get("decay_start_frac", 0.8)
        assert 0.0 < frac < 1.0, "decay_start_frac must be between 0 and 1"
        start_step = int(frac * T)
        if step < start_step:
            return base
        return base * max((T - step) / max(1, T - start_step), 0.0)
    raise ValueError(f"unknown lr_scheduler {kind!r}")


def _stack_layers(batch: Dict[int, torch.Tensor], layers) -> torch.Tensor:
    stacked = getattr(batch, "stacked", None)
    if stacked is not None:
        return stacked
    return torch.stack([batch[l] for l in layers])


class CLTTrainer:
    def __init__(
        self,
        clt_config: CLTConfig,
        training_config: TrainingConfig,
        log_dir: Optional[str] = None,
        device: Optional[Any] = None,
        distributed: bool = False,
        resume_from_checkpoint_path: Optional[str] = None,
        activation_store: Optional[BaseActivationStore] = None,
    ):
        self.clt_config = clt_config
        self.training_config = training_config
        self.distributed = distributed
        self.rank, self.world_size, self.local_rank = 0, 1, 0
        self.process_group = None
        self._owns_process_group = False

        if distributed:
            if not dist.is_initialized():
                if torch.cuda.is_available():
                    # bound to this rank's device from the start (eager communicator): the configuration that the symmetric-memory
                    # exchange and the sharded staging are run with everywhere else
                    local = int(os.environ.get("LOCAL_RANK", "0"))
                    torch.cuda.set_device(local)
                    dist.init_process_group(backend="nccl", device_id=torch.device(f"cuda:{local}"))
                else:
                    dist.init_process_group(backend="gloo")
                self._owns_process_group = True
            self.rank, self.world_size = dist.get_rank(), dist.get_world_size()
            self.local_rank = int(os.environ.get("LOCAL_RANK", self.rank))
            if torch.cuda.is_available():
                device = torch.device(f"cuda:{self.local_rank}")
                torch.cuda.set_device(device)
            else:
                device = torch.device("cpu")
            self.process_group = dist.group.WORLD
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)

        # mixed precision: autocast for fp16/bf16, loss scaling for fp16 only (reference trainer.py:107-141)
        prec = training_config.precision
        self.autocast_enabled = prec in ("fp16", "bf16") and self.device.type in ("cuda", "cpu")
        self.autocast_dtype = {"fp16": torch.float16, "bf16": torch.bfloat16}.get(prec, torch.float32)
        if self.device.type == "cpu" and prec == "fp16":
            self.autocast_enabled = False
        self.scaler = torch.amp.GradScaler(self.device.type, enabled=(prec == "fp16" and self.device.type == "cuda"))

        self.log_dir = log_dir or f"clt_train_{int(time.time())}"
        if self.rank == 0:
            os.makedirs(self.log_dir, exist_ok=True)
        self.start_time = time.time()

        seed = training_config.seed + self.rank  # reference: per-rank seed (trainer.py:155-157)
        torch.manual_seed(seed)
        np.random.seed(seed % (2 ** 32))
        random.seed(seed)

        self.profiler = TrainingProfiler(enabled=training_config.enable_profiling, log_interval=training_config.log_interval)
        self.memory_profiler = CUDAMemoryProfiler(enabled=training_config.enable_profiling)
        self.dist_profiler = DistributedProfiler(enabled=training_config.enable_profiling and distributed, rank=self.rank)

        self.model = CrossLayerTranscoder(clt_config, process_group=self.process_group, device=self.device, profiler=self.profiler)
        if prec == "fp16" and training_config.fp16_convert_weights:
            self.model.half()
            self.model.dtype = torch.float16

        # --- data
        self.activation_store = activation_store if activation_store is not None else self._create_activation_store()
        mean_tg = getattr(self.activation_store, "mean_tg", {}) or {}
        std_tg = getattr(self.activation_store, "std_tg", {}) or {}
        self.loss_manager = LossManager(training_config, mean_tg=mean_tg, std_tg=std_tg, clt_config=clt_config)
        self.evaluator = CLTEvaluator(
            self.model, self.device, self.start_time, mean_tg=mean_tg, std_tg=std_tg,
            normalization_method=training_config.normalization_method, d_model=clt_config.d_model,
        )

        # --- step implementation
        self.engine = None
        self.optimizer = None
        self._select_engine(mean_tg, std_tg)

        # dead-feature counter, sharded with the features: [L, valid_features]
        L = clt_config.num_layers
        if self.engine is None:
            self.n_forward_passes_since_fired = torch.zeros(L, self.model.valid_features, dtype=torch.long, device=self.device)
        async_ckpt = training_config.async_checkpoint
        if async_ckpt is None:
            async_ckpt = self.device.type == "cuda"
        self.checkpoint_manager = CheckpointManager(
            self.model, self.activation_store, None, self.log_dir, distributed, self.rank, self.device, self.world_size,
            async_save=bool(async_ckpt),
        )
        self._resume_state: Optional[Dict[str, Any]] = None
        self.start_step = 0
        resume_wandb_id = None
        if resume_from_checkpoint_path:
            self._resume_state = self.checkpoint_manager.load_checkpoint(resume_from_checkpoint_path)
            resume_wandb_id = (self._resume_state or {}).get("wandb_run_id")
        if training_config.enable_wandb and self.rank == 0:
            self.wandb_logger: Any = WandBLogger(training_config, clt_config, self.log_dir, resume_wandb_id)
        else:
            self.wandb_logger = DummyWandBLogger()
        self.checkpoint_manager.wandb_logger = self.wandb_logger
        self.metric_logger = MetricLogger(distributed, self.rank, self.log_dir, self.wandb_logger, training_config, self.world_size)
        if self._resume_state:
            self._apply_resume_state(self._resume_state)

    # ------------------------------------------------------------------ setup helpers
    def _create_activation_store(self) -> BaseActivationStore:
        from .data.activation_store_factory import create_activation_store

        return create_activation_store(
            self.training_config, self.clt_config, self.device, rank=self.rank, world=self.world_size,
            shard_data=not self.distributed,
            shard_group=self.process_group if (self.distributed and self.world_size > 1 and self.device.type == "cuda") else None,
        )

    def _select_engine(self, mean_tg, std_tg) -> None:
        from .fused_engine import FusedBatchTopKEngine, engine_supports

        tc = self.training_config
        want = tc.engine
        reason = None
        if want == "autograd":
            reason = "engine='autograd' requested"
        elif self.device.type != "cuda":
            reason = "no CUDA device"
        else:
            reason = engine_supports(self.clt_config, tc, self.model)
            if reason is None and want == "auto" and self.clt_config.activation_fn in ("jumprelu", "relu"):
                # the fused threshold step keeps the active entries in lists of fused_max_active_per_token per token; whether
                # a run is sparse enough for them is decided on its first batch (see _probe_density)
                self._probe_pending = True
            if reason is None and self.world_size > 1:
                from ..parallel.symm import SymmetricExchange

                self._symm = SymmetricExchange.create(self.process_group, self.device, self.clt_config, tc.train_batch_size_tokens)
        if reason is None:
            sigma = None
            if tc.normalization_method == "mean_std" and std_tg:
                sigma = torch.stack([std_tg[l].reshape(-1).float() for l in range(self.clt_config.num_layers)])
            elif tc.normalization_method == "sqrt_d_model":
                sigma = torch.full((self.clt_config.num_layers, self.clt_config.d_model), 1.0 / math.sqrt(self.clt_config.d_model))
            self.engine = FusedBatchTopKEngine(self.model, tc, tc.train_batch_size_tokens, sigma_tg=sigma,
                                               symm=getattr(self, "_symm", None))
            logger.info("Rank %d: using the fused sm_100a step engine", self.rank)
            if not getattr(self, "_probe_pending", False):
                self._restrict_target_staging()  # while the first batch may still send the run to the autograd step, every row travels
            self._gate_staging()
            return
        if want == "fused":
            raise ValueError(f"engine='fused' requested but not available: {reason}")
        logger.info("Rank %d: using the autograd step (%s)", self.rank, reason)
        self._build_autograd_optimizer()

    def _restrict_target_staging(self) -> None:
        """Tensor-parallel fused runs: the loss of a token is finished by the rank that owns its row block, which is the
        block that rank's stager loads from the host, so the targets need not travel to the peers (half of the staging
        traffic over NVLink).  Evaluation gathers the owners' target rows again (``_full_targets``)."""
        self._target_rows = None
        stager = getattr(self.activation_store, "stager", None)
        if self.world_size <= 1 or stager is None or getattr(stager, "shard_world", 1) != self.world_size:
            return
        B = self.training_config.train_batch_size_tokens
        symm = getattr(self, "_symm", None)
        if symm is None or B % self.world_size != 0 or symm.rows_per_rank != getattr(stager, "rows_per_rank", -1):
            return
        if getattr(stager, "shard_rank", -1) != self.rank:
            return
        if stager.push_only_leading(self.clt_config.num_layers):
            self._target_rows = (self.rank * symm.rows_per_rank, symm.rows_per_rank)

    def _gate_staging(self) -> None:
        """Lets the store's staging copies start when a step reaches its optimizer sweep instead of at the step boundary:
        host-to-device writes that arrive during the read-streaming kernels at the start of a step (column statistics,
        selection pass) slow those by far more than their own volume; the sweep mixes reads and writes anyway."""
        stager = getattr(self.activation_store, "stager", None)
        if stager is None or not getattr(stager, "cuda", False) or not hasattr(stager, "gate"):
            return
        eng = self.engine
        eng.sweep_begin = torch.cuda.Event()
        eng.sweep_begin.record()
        stager.gate = lambda: eng.sweep_begin

    def _full_targets(self, Y: torch.Tensor) -> torch.Tensor:
        """``[L, B, d]`` targets with every rank's owned rows filled in (all-gather over the process group)."""
        if getattr(self, "_target_rows", None) is None:
            return Y
        import torch.distributed as dist

        r0, n = self._target_rows
        L, B, d = Y.shape
        own = Y[:, r0:r0 + n].contiguous()
        parts = [torch.empty_like(own) for _ in range(self.world_size)]
        dist.all_gather(parts, own, group=self.process_group)  # list form: available on every backend
        return torch.cat(parts, dim=1)[:, :B].contiguous()

    def _build_autograd_optimizer(self) -> None:
        tc = self.training_config
        kwargs: Dict[str, Any] = {"lr": tc.learning_rate}
        if tc.optimizer_beta1 is not None or tc.optimizer_beta2 is not None:
            kwargs["betas"] = (tc.optimizer_beta1 if tc.optimizer_beta1 is not None else 0.9,
                               tc.optimizer_beta2 if tc.optimizer_beta2 is not None else 0.999)
        opt_cls = torch.optim.Adam if tc.optimizer == "adam" else torch.optim.AdamW
        self.optimizer = opt_cls(self.model.parameters(), **kwargs)

    # ------------------------------------------------------------------ dead features
    @property
    def dead_neurons_mask(self) -> torch.Tensor:
        """``[L, valid_features]`` boolean mask of this rank's features that did not fire for more than
        ``dead_feature_window`` steps."""
        window = self.training_config.dead_feature_window
        if self.engine is not None:
            c = self.engine.dead_counter.view(self.clt_config.num_layers, self.model.local_features)
            return (c[:, : self.model.valid_features] > window).detach()
        return (self.n_forward_passes_since_fired > window).detach()

    @torch.no_grad()
    def _update_dead_counters(self, acts: Dict[int, torch.Tensor]) -> None:
        for l, a in acts.items():
            if a.numel() == 0 or l >= self.n_forward_passes_since_fired.shape[0]:
                continue
            fired = (a.detach() > 1e-6).any(dim=0)[: self.n_forward_passes_since_fired.shape[1]]
            self.n_forward_passes_since_fired[l] += 1
            self.n_forward_passes_since_fired[l][fired] = 0

    # ------------------------------------------------------------------ one step
    def _next_batch(self):
        try:
            return next(self.activation_store)
        except StopIteration:
            if self.training_config.auto_advance_epoch and hasattr(self.activation_store, "advance_epoch"):
                self.activation_store.advance_epoch()
                return next(self.activation_store)
            raise

    def train_step(self, inputs: Dict[int, torch.Tensor], targets: Dict[int, torch.Tensor], step: int) -> Dict[str, torch.Tensor]:
        """One optimisation step; returns the loss terms as device scalars (no host sync)."""
        tc = self.training_config
        lr = learning_rate_at(tc, step)
        if self.engine is not None and getattr(self, "_probe_pending", False):
            self._probe_density(inputs)
        if self.engine is not None:
            return self._train_step_fused(inputs, targets, step, lr)
        return self._train_step_autograd(inputs, targets, step, lr)

    def _probe_density(self, inputs) -> None:
        """engine="auto" with JumpReLU / ReLU: one selection pass over the first batch decides between the two step
        implementations.  The fused step holds at most ``fused_max_active_per_token`` active entries per token; a model
        that starts denser than half of that (the reference's default threshold 0.03 on unit-variance inputs does) takes
        the autograd step, whose dense kernels are the better fit there.  All ranks take the same branch."""
        self._probe_pending = False
        eng, tc = self.engine, self.training_config
        layers = list(range(self.clt_config.num_layers))
        X = _stack_layers(inputs, layers).to(eng.t16)
        eng.encode_select(X)
        per_token = (eng.ctl[3].float() / eng.B).reshape(1)
        if self.world_size > 1:
            pops.all_reduce(per_token, group=self.process_group)
        too_dense = torch.tensor([float(per_token.item()) > 0.5 * tc.fused_max_active_per_token or int(eng.status[0].item()) != 0],
                                 dtype=torch.int32, device=self.device)
        if self.world_size > 1:
            pops.all_reduce(too_dense, op=pops.MAX, group=self.process_group)
        eng.status.zero_()
        eng.fired.zero_()
        if bool(too_dense.item()):
            logger.info("Rank %d: %.0f active features per token on the first batch: using the autograd step", self.rank, float(per_token.item()))
            self.engine = None
            stager = getattr(self.activation_store, "stager", None)
            if stager is not None and hasattr(stager, "gate"):
                stager.gate = None
            self._build_autograd_optimizer()
            self.n_forward_passes_since_fired = torch.zeros(self.clt_config.num_layers, self.model.valid_features, dtype=torch.long, device=self.device)
        else:
            self._restrict_target_staging()  # batches staged from here on carry the targets of the owned token rows only

    def _train_step_fused(self, inputs, targets, step: int, lr: float) -> Dict[str, torch.Tensor]:
        tc, eng = self.training_config, self.engine
        layers = list(range(self.clt_config.num_layers))
        with self.profiler.timer("forward_pass"):
            X = _stack_layers(inputs, layers)
            Y = _stack_layers(targets, layers)
            if X.dtype != eng.t16:
                X, Y = X.to(eng.t16), Y.to(eng.t16)
        lam = sparsity_lambda_at(tc, step, tc.training_steps)
        if self.clt_config.activation_fn == "batchtopk" and not tc.apply_sparsity_penalty_to_batchtopk:
            lam = 0.0
        self.loss_manager.current_sparsity_lambda = lam
        # a feature is dead once its counter passed the window, which cannot happen before `dead_feature_window` steps
        # unless the counters were restored from a checkpoint: the counters alone decide
        need_aux = bool(tc.aux_loss_factor) and self.clt_config.activation_fn in ("batchtopk", "topk") and self._any_dead_cached(step)
        pre_coef = tc.preactivation_coef if tc.preactivation_coef is not None else 0.0
        with self.profiler.timer("optimizer_step"):
            out = eng.train_step(
                X, Y, step, lr, sparsity_lambda=lam, preactivation_coef=pre_coef,
                aux_factor=(tc.aux_loss_factor if need_aux else 0.0), dead_window=(tc.dead_feature_window if need_aux else None),
            )
        return out.as_dict()

    def _any_dead_cached(self, step: int) -> bool:
        """True when any rank holds a dead feature.  One host read every 100 steps is enough (features die
        slowly).  The answer is agreed over the process group (all-reduce MAX at the same steps on every rank):
        the auxiliary term runs collectives, so every rank has to take the same branch."""
        if not hasattr(self, "_dead_seen") or step % 100 == 0:
            per_layer = self.dead_neurons_mask.sum(dim=1).to(torch.int32)
            count = per_layer.max().reshape(1)  # largest per-layer dead count of any shard
            if self.world_size > 1:
                pops.all_reduce(count, op=pops.MAX, group=self.process_group)
                pops.all_reduce(per_layer, group=self.process_group)  # per layer over all shards
            n, n_all = int(count.item()), int(per_layer.max().item())
            self._dead_seen = n_all > 0
            if self.engine is not None:
                self.engine.set_dead_count_hint(n, n_all)  # sizes the compact dead set of the fused auxiliary term
        return self._dead_seen

    def _train_step_autograd(self, inputs, targets, step: int, lr: float) -> Dict[str, torch.Tensor]:
        tc = self.training_config
        for g in self.optimizer.param_groups:
            g["lr"] = lr
        self.optimizer.zero_grad(set_to_none=True)
        with torch.autocast(device_type=self.device.type, dtype=self.autocast_dtype, enabled=self.autocast_enabled):
            with self.profiler.timer("forward_pass"):
                pass
            with self.profiler.timer("loss_computation"):
                loss, parts, acts = self.loss_manager.compute_total_loss_tensors(
                    self.model, inputs, targets, step, tc.training_steps, dead_neuron_mask=self.dead_neurons_mask
                )
        with self.profiler.timer("dead_neuron_update"):
            self._update_dead_counters(acts)
        if tc.debug_anomaly:
            torch.autograd.set_detect_anomaly(True)
        finite = torch.isfinite(loss.detach())
        with self.profiler.timer("backward_pass"):
            self.scaler.scale(loss).backward()
        self.scaler.unscale_(self.optimizer)
        # replicated parameters see bit-identical gradients on every rank (same replicated
        # reconstruction, same order of operations), so no gradient all-reduce is needed here
        if tc.gradient_clip_val is not None:
            with self.profiler.timer("gradient_clipping"):
                self._clip_grad_norm(tc.gradient_clip_val)
        with self.profiler.timer("optimizer_step"):
            if self.device.type == "cpu" or not self.scaler.is_enabled():
                # skip the update on a non-finite loss (reference: NaN-loss skip, trainer.py:740-747)
                if bool(finite):
                    self.optimizer.step()
            else:
                self.scaler.step(self.optimizer)
        self.scaler.update()
        self.model.invalidate_decoder_norms()
        return parts

    def _clip_grad_norm(self, max_norm: float) -> None:
        """Global-norm clipping.  Sharded parameters contribute their shard's squared norm, summed over
        ranks; replicated parameters are counted once (the reference clips with the local norm only)."""
        from ..models.base import is_replicated

        sq_sharded = torch.zeros((), device=self.device)
        sq_repl = torch.zeros((), device=self.device)
        params = [p for p in self.model.parameters() if p.grad is not None]
        for p in params:
            s = p.grad.detach().float().pow(2).sum()
            if is_replicated(p):
                sq_repl = sq_repl + s
            else:
                sq_sharded = sq_sharded + s
        if self.world_size > 1:
            pops.all_reduce(sq_sharded, group=self.process_group)
        total = (sq_sharded + sq_repl).sqrt()
        coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
        for p in params:
            p.grad.mul_(coef.to(p.grad.dtype))

    # ------------------------------------------------------------------ training loop
    def train(self, eval_every: Optional[int] = None) -> CrossLayerTranscoder:
        tc = self.training_config
        if self.rank == 0:
            logger.info("Training CLT: %d steps, batch %d tokens, %d rank(s), device %s",
                        tc.training_steps, tc.train_batch_size_tokens, self.world_size, self.device)
        self._save_run_config()
        step = self.start_step
        last_parts = None
        health = None
        lost_peer = False
        if self.world_size > 1 and tc.peer_health_timeout_s:
            from ..parallel.health import HeartbeatMonitor

            health = HeartbeatMonitor(dist.distributed_c10d._get_default_store(), self.rank, self.world_size,
                                      timeout_s=float(tc.peer_health_timeout_s))
        try:
            for step in range(self.start_step, tc.training_steps):
                if health is not None:
                    health.ready(step)  # raises PeerLostError before anything of this step is launched
                with self.profiler.timer("data_loading"):
                    try:
                        inputs, targets = self._next_batch()
                    except StopIteration:
                        if self.rank == 0:
                            logger.info("Activation store exhausted. Training finished early.")
                        pops.barrier(self.process_group)
                        break
                if not inputs or not any(v.numel() > 0 for v in inputs.values()):
                    logger.warning("Rank %d: empty batch at step %d, skipping", self.rank, step)
                    continue
                parts = self.train_step(inputs, targets, step)
                last_parts = parts
                self.metric_logger.log_training_step(
                    step, parts, current_lr=learning_rate_at(tc, step),
                    current_sparsity_lambda=self.loss_manager.get_current_sparsity_lambda(),
                )
                self.profiler.step()
                last = step == tc.training_steps - 1
                if step % tc.eval_interval == 0 or last:
                    self._run_evaluation(step, inputs, targets)
                want_ckpt = (step > 0 and step % tc.checkpoint_interval == 0) or last
                if self.engine is not None and (want_ckpt or step % max(1, tc.log_interval) == 0):
                    # before anything of this step is written out: a step whose kernels gave up a wait (or ran out
                    # of list capacity) skipped its update, and the run stops here instead of saving it as good
                    self._check_device_status()
                if want_ckpt:
                    self.save_checkpoint(step)
        except KeyboardInterrupt:
            if self.rank == 0:
                logger.warning("Interrupted at step %d; writing the final checkpoint", step)
        except BaseException as exc:
            from .fused_engine import EngineStatusError

            if health is not None:
                from ..parallel.health import PeerLostError

                if not isinstance(exc, PeerLostError):
                    health.leave(f"{type(exc).__name__} at step {step}")
                # a collective with a lost rank would never complete: skip the final barrier and checkpoint
                logger.error("Rank %d: stopping at step %d: %s", self.rank, step, exc)
                lost_peer = True
            if isinstance(exc, EngineStatusError):
                # this rank's kernels reported a failed step: the other ranks may not have seen one, so no collective
                # is entered here, and the weights of a failed step are not written over the last good checkpoint
                logger.error("Rank %d: stopping at step %d without a final checkpoint: %s", self.rank, step, exc)
                lost_peer = True
            raise
        finally:
            if not lost_peer:
                pops.barrier(self.process_group)
                self.save_checkpoint(step, final=True)
            self.checkpoint_manager.wait()
            if hasattr(self.activation_store, "close"):
                self.activation_store.close()
            self.metric_logger._save_metrics_to_disk()
            self._save_run_config()
            if self.rank == 0:
                os.makedirs(os.path.join(self.log_dir, "final"), exist_ok=True)
                self.wandb_logger.log_artifact(os.path.join(self.log_dir, "final"), "model", "final")
            self.wandb_logger.finish()
            self.profiler.log_summary()
            self.memory_profiler.log_summary()
            self.dist_profiler.log_summary()
            if self._owns_process_group and dist.is_initialized():
                dist.destroy_process_group()
        return self.model

    def _check_device_status(self) -> None:
        self.engine.check_status()
        stager = getattr(self.activation_store, "stager", None)
        if stager is not None and hasattr(stager, "check_status"):
            stager.check_status()

    def _run_evaluation(self, step: int, inputs, targets) -> None:
        tc = self.training_config
        pops.barrier(self.process_group)
        # fused runs evaluate through the sparse forward (no dense [B, F] activations) unless the dense diagnostics
        # were asked for; the dead-feature counters are not touched by an evaluation forward
        fused_eval = self.engine is not None and not tc.compute_sparsity_diagnostics
        if getattr(self, "_target_rows", None) is not None and not fused_eval:
            layers = list(range(self.clt_config.num_layers))
            full = self._full_targets(_stack_layers(targets, layers))
            targets = {l: full[l] for l in layers}
        with self.profiler.timer("evaluation"):
            if fused_eval:
                layers = list(range(self.clt_config.num_layers))
                X, Y = _stack_layers(inputs, layers), self._full_targets(_stack_layers(targets, layers))
                if X.dtype != self.engine.t16:
                    X, Y = X.to(self.engine.t16), Y.to(self.engine.t16)
                metrics = self.evaluator.compute_metrics_from_engine(self.engine, X, Y, dead_neuron_mask=self.dead_neurons_mask)
            else:
                autocast = torch.autocast(device_type=self.device.type, dtype=self.autocast_dtype, enabled=self.autocast_enabled)
                with autocast, torch.no_grad():
                    metrics = self.evaluator.compute_metrics(inputs, targets, dead_neuron_mask=self.dead_neurons_mask)
                    # per-layer std of the pre-activations (reference trainer.py:884-897)
                    pre, _ = self.model._encode_all_layers(inputs, gather=False)
                    stds = torch.stack([p.float().std() if p.numel() > 1 else torch.zeros((), device=self.device) for p in pre.values()])
                    metrics["layerwise/preactivation_std_dev"] = {f"layer_{l}": v for l, v in zip(pre.keys(), stds.tolist())}
                    if tc.compute_sparsity_diagnostics:
                        from .diagnostics import compute_sparsity_diagnostics

                        acts = self.model.get_feature_activations(inputs, gather=False)
                        metrics.update(compute_sparsity_diagnostics(self.model, tc, acts))
        self.metric_logger.log_evaluation_metrics(step, metrics)
        if self.rank == 0:
            from ..utils import format_elapsed_time

            logger.info(
                "step %d [%s]: NMSE %.4f, EV %.4f, avg L0 %.1f, dead %d",
                step, format_elapsed_time(time.time() - self.start_time),
                metrics.get("reconstruction/normalized_mean_reconstruction_error", float("nan")),
                metrics.get("reconstruction/explained_variance", float("nan")), metrics.get("sparsity/avg_l0", float("nan")),
                metrics.get("dead_features/total_eval", 0),
            )
        pops.barrier(self.process_group)

    # ------------------------------------------------------------------ checkpoint / resume
    def _trainer_state(self, step: int) -> Dict[str, Any]:
        state: Dict[str, Any] = {
            "step": step,
            "scaler_state_dict": self.scaler.state_dict() if self.scaler.is_enabled() else None,
            "wandb_run_id": self.wandb_logger.get_current_wandb_run_id(),
            "torch_rng_state": torch.get_rng_state(),
            "numpy_rng_state": np.random.get_state(),
            "python_rng_state": random.getstate(),
            "engine": "fused" if self.engine is not None else "autograd",
            "world_size": self.world_size,
        }
        if torch.cuda.is_available() and self.device.type == "cuda":
            state["cuda_rng_state"] = torch.cuda.get_rng_state(self.device)
        if self.engine is None:
            state["n_forward_passes_since_fired"] = self.n_forward_passes_since_fired.cpu()
        return state

    def _optimizer_tensors(self) -> Dict[str, torch.Tensor]:
        if self.engine is not None:
            return dict(self.engine.optimizer_state_dict())
        out: Dict[str, torch.Tensor] = {}
        # this rank's dead-feature counters travel with its optimizer shard (the pickled trainer state is rank 0's)
        pad = self.model.local_features - self.n_forward_passes_since_fired.shape[1]
        out["dead_counter_2d"] = torch.nn.functional.pad(self.n_forward_passes_since_fired, (0, pad)) if pad else self.n_forward_passes_since_fired
        names = {id(p): n for n, p in self.model.named_parameters()}
        for p, st in self.optimizer.state.items():
            n = names.get(id(p))
            if n is None:
                continue
            for k, v in st.items():
                out[f"{n}::{k}"] = v if isinstance(v, torch.Tensor) else torch.tensor(float(v))
        return out

    def _load_optimizer_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.engine is not None:
            self.engine.load_optimizer_state_dict({k: v.to(self.device) for k, v in tensors.items()})
            return
        params = dict(self.model.named_parameters())
        for key, v in tensors.items():
            if key == "dead_counter_2d":
                self.n_forward_passes_since_fired.copy_(v[:, : self.n_forward_passes_since_fired.shape[1]].to(self.device))
                self._dead_counter_restored = True
                continue
            if "::" not in key:
                continue
            name, field = key.split("::", 1)
            p = params.get(name)
            if p is None:
                continue
            st = self.optimizer.state[p]
            st[field] = v.to(self.device if field != "step" else "cpu") if v.dim() > 0 or field != "step" else v.clone()

    def save_checkpoint(self, step: int, final: bool = False) -> None:
        with self.profiler.timer("checkpoint"):
            self.checkpoint_manager._save_checkpoint(step, self._trainer_state(step), self._optimizer_tensors())

    def _apply_resume_state(self, state: Dict[str, Any]) -> None:
        if "optimizer_tensors" in state:
            self._load_optimizer_tensors(state["optimizer_tensors"])
        if state.get("scaler_state_dict") and self.scaler.is_enabled():
            self.scaler.load_state_dict(state["scaler_state_dict"])
        if self.engine is None and state.get("n_forward_passes_since_fired") is not None and not getattr(self, "_dead_counter_restored", False):
            c = state["n_forward_passes_since_fired"].to(self.device)
            if c.shape == self.n_forward_passes_since_fired.shape:
                self.n_forward_passes_since_fired.copy_(c)
        if state.get("torch_rng_state") is not None:
            torch.set_rng_state(state["torch_rng_state"].cpu() if isinstance(state["torch_rng_state"], torch.Tensor) else state["torch_rng_state"])
        if state.get("cuda_rng_state") is not None and self.device.type == "cuda":
            torch.cuda.set_rng_state(state["cuda_rng_state"].cpu(), self.device)
        if state.get("numpy_rng_state") is not None:
            np.random.set_state(state["numpy_rng_state"])
        if state.get("python_rng_state") is not None:
            random.setstate(state["python_rng_state"])
        self.start_step = int(state.get("step", -1)) + 1
        self.model.invalidate_decoder_norms()
        logger.info("Rank %d: resuming from step %d", self.rank, self.start_step)

    def _save_run_config(self) -> None:
        if self.rank != 0:
            return
        cfg = dataclasses.asdict(self.clt_config)
        cfg["normalization_method"] = self.training_config.normalization_method
        cfg["expected_input_dtype"] = self.training_config.activation_dtype
        try:
            with open(os.path.join(self.log_dir, "cfg.json"), "w") as fh:
                json.dump(cfg, fh, indent=2)
            with open(os.path.join(self.log_dir, "training_config.json"), "w") as fh:
                json.dump(dataclasses.asdict(self.training_config), fh, indent=2)
        except OSError as exc:
            logger.warning("could not write run configuration: %s", exc)
