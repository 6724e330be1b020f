"""Model, training and inference configuration dataclasses.

Field names, defaults and JSON layout follow the reference configuration
(clt/config/clt_config.py:10-311) so that existing ``cfg.json`` files and CLI
flags keep working.  Differences that are deliberate:

* ``normalization_method="auto"`` (and the other legacy spellings) is accepted
  everywhere and folded to ``mean_std`` / ``sqrt_d_model`` (the reference only
  folds it in ``CLTConfig.from_json`` and rejects it in ``TrainingConfig``).
* ``optimizer_states_dtype`` and ``enable_stochastic_rounding`` are live: the
  fused Adam kernel keeps fp32 moments for bf16 weights (``"model_dtype"`` and
  ``"float32"``; the reference's torch optimizer would keep bf16 moments for bf16
  parameters) and can round the updated weight stochastically;
  ``optimizer_states_dtype="bfloat16"`` stores the moments of the encoder and
  decoder weights in bf16 with stochastic rounding (fused step, untied decoders).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

ACTIVATION_FNS = ("jumprelu", "relu", "batchtopk", "topk")
NORM_METHODS = ("none", "mean_std", "sqrt_d_model")
DECODER_TYING = ("none", "per_source", "per_target")

_LEGACY_NORM = {
    "auto": "mean_std",
    "estimated_mean_std": "mean_std",
    "auto_sqrt_d_model": "sqrt_d_model",
    "estimated_mean_std_sqrt_d_model": "sqrt_d_model",
}


def canonical_normalization(name: Optional[str]) -> str:
    """Map legacy normalisation names onto the three canonical ones."""
    if name is None:
        return "none"
    return _LEGACY_NORM.get(name, name)


@dataclass
class CLTConfig:
    """Architecture of a cross-layer transcoder (reference: clt_config.py:10-76)."""

    num_features: int
    num_layers: int
    d_model: int
    model_name: Optional[str] = None
    normalization_method: str = "none"
    activation_fn: str = "jumprelu"
    jumprelu_threshold: float = 0.03
    batchtopk_k: Optional[int] = None
    batchtopk_straight_through: bool = True
    topk_k: Optional[float] = None
    topk_straight_through: bool = True
    topk_mode: str = "global"
    clt_dtype: Optional[str] = None
    expected_input_dtype: Optional[str] = None
    mlp_input_template: Optional[str] = None
    mlp_output_template: Optional[str] = None
    tl_input_template: Optional[str] = None
    tl_output_template: Optional[str] = None
    decoder_tying: str = "none"
    enable_feature_offset: bool = False
    enable_feature_scale: bool = False
    skip_connection: bool = False

    def __post_init__(self) -> None:
        self.normalization_method = canonical_normalization(self.normalization_method)
        assert self.num_features > 0, "Number of features must be positive"
        assert self.num_layers > 0, "Number of layers must be positive"
        assert self.d_model > 0, "Model dimension must be positive"
        assert self.normalization_method in NORM_METHODS, (
            f"Invalid normalization_method: {self.normalization_method}. Must be one of {list(NORM_METHODS)}"
        )
        assert self.activation_fn in ACTIVATION_FNS, (
            f"Invalid activation_fn: {self.activation_fn}. Must be one of {list(ACTIVATION_FNS)}"
        )
        assert self.decoder_tying in DECODER_TYING, (
            f"Invalid decoder_tying: {self.decoder_tying}. Must be one of {list(DECODER_TYING)}"
        )
        assert self.topk_mode in ("global", "per_layer"), f"Invalid topk_mode: {self.topk_mode}"
        if self.activation_fn == "batchtopk":
            if self.batchtopk_k is None:
                raise ValueError("batchtopk_k must be specified for BatchTopK.")
            if self.batchtopk_k <= 0:
                raise ValueError("batchtopk_k must be positive.")
        if self.activation_fn == "topk":
            if self.topk_k is None:
                raise ValueError("topk_k must be specified for TopK activation function.")
            if self.topk_k <= 0:
                raise ValueError("topk_k must be positive if specified.")

    # -- JSON round trip (reference: clt_config.py:78-124) ------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "CLTConfig":
        d = dict(raw)
        if d.pop("sqrt_d_model_normalize", False):
            d["normalization_method"] = "sqrt_d_model"
        known = {f.name for f in dataclasses.fields(cls)}
        # Run directories written by the trainer add training-side keys to cfg.json;
        # keep the ones that are model fields and drop the rest.
        d = {k: v for k, v in d.items() if k in known}
        return cls(**d)

    @classmethod
    def from_json(cls, json_path: str) -> "CLTConfig":
        with open(json_path, "r") as fh:
            return cls.from_dict(json.load(fh))

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def to_json(self, json_path: str) -> None:
        with open(json_path, "w") as fh:
            json.dump(self.to_dict(), fh, indent=4)


@dataclass
class TrainingConfig:
    """Training hyper-parameters (reference: clt_config.py:127-269)."""

    learning_rate: float
    training_steps: int
    seed: int = 42
    gradient_clip_val: Optional[float] = None
    train_batch_size_tokens: int = 4096
    n_batches_in_buffer: int = 16
    precision: str = "fp32"
    fp16_convert_weights: bool = False
    debug_anomaly: bool = False
    normalization_method: str = "mean_std"
    normalization_estimation_batches: int = 50
    activation_source: str = "local_manifest"
    activation_dtype: str = "bfloat16"
    activation_path: Optional[str] = None
    remote_config: Optional[Dict[str, Any]] = None
    sampling_strategy: str = "sequential"
    sparsity_lambda: float = 1e-3
    sparsity_lambda_schedule: str = "linear"
    sparsity_lambda_delay_frac: float = 0.1
    sparsity_c: float = 1.0
    preactivation_coef: float = 3e-6
    aux_loss_factor: Optional[float] = None
    apply_sparsity_penalty_to_batchtopk: bool = True
    optimizer: str = "adamw"
    optimizer_beta1: Optional[float] = None
    optimizer_beta2: Optional[float] = None
    optimizer_states_dtype: str = "model_dtype"
    enable_stochastic_rounding: bool = False
    lr_scheduler: Optional[str] = "linear"
    lr_scheduler_params: Optional[Dict[str, Any]] = None
    log_interval: int = 100
    eval_interval: int = 1000
    checkpoint_interval: int = 1000
    diag_every_n_eval_steps: Optional[int] = None
    max_features_for_diag_hist: Optional[int] = None
    compute_sparsity_diagnostics: bool = False
    enable_profiling: bool = False
    dead_feature_window: int = 1000
    enable_wandb: bool = False
    wandb_project: Optional[str] = None
    wandb_entity: Optional[str] = None
    wandb_run_name: Optional[str] = None
    wandb_tags: Optional[list] = field(default_factory=list)
    jumprelu_default_theta_on_convert: float = 1e6
    # --- additions of this framework (absent from the reference) -----------
    # Use the fused sm_100a step engine when the model/loss combination is
    # covered by it; "auto" falls back to the autograd path otherwise.
    engine: str = "auto"
    # Number of batches the activation store keeps in flight (pinned host ring
    # + side-stream copies).  The reference never enables its prefetch thread.
    prefetch_batches: int = 2
    # Wrap around to a new epoch (seed + epoch) when the store is exhausted
    # instead of ending training early.
    auto_advance_epoch: bool = True
    # Tensor-parallel jobs: seconds after which a rank that has not announced the next step is declared
    # lost (host-side heartbeat through the job's store, checked before every launch).  None: off.
    peer_health_timeout_s: Optional[float] = None
    # Fused JumpReLU step: capacity of the active-entry lists, in entries per token (a step whose
    # activations are denser reports it through the status word).
    fused_max_active_per_token: int = 1024
    # Checkpoints: copy device -> pinned host on a side stream and write the files from a background thread
    # (None: on for CUDA runs, off on CPU).
    async_checkpoint: Optional[bool] = None
    # fp16 loss scaling of the fused step (same defaults as torch.amp.GradScaler, reference trainer.py:107-141)
    loss_scale_init: float = 65536.0
    loss_scale_growth_interval: int = 2000

    def __post_init__(self) -> None:
        self.normalization_method = canonical_normalization(self.normalization_method)
        assert self.learning_rate > 0, "Learning rate must be positive"
        assert self.training_steps > 0, "Training steps must be positive"
        assert self.train_batch_size_tokens > 0, "Training batch size (tokens) must be positive"
        assert self.n_batches_in_buffer > 0, "Buffer size must be positive"
        assert self.sparsity_lambda >= 0, "Sparsity lambda must be non-negative"
        assert self.dead_feature_window > 0, "Dead feature window must be positive"
        assert self.precision in ("fp32", "fp16", "bf16"), f"Invalid precision: {self.precision}"
        if self.activation_source == "local_manifest":
            assert self.activation_path is not None, (
                "activation_path must be specified when activation_source is 'local_manifest'"
            )
        elif self.activation_source == "remote":
            assert self.remote_config is not None, (
                "remote_config dict must be provided when activation_source is 'remote'"
            )
            assert "server_url" in self.remote_config and "dataset_id" in self.remote_config, (
                "remote_config must contain 'server_url' and 'dataset_id'"
            )
        else:
            raise ValueError(f"Unsupported activation_source: {self.activation_source}")
        assert self.sampling_strategy in ("sequential", "random_chunk"), (
            "sampling_strategy must be 'sequential' or 'random_chunk'"
        )
        assert self.sparsity_lambda_schedule in ("linear", "delayed_linear"), "Invalid sparsity_lambda_schedule"
        if self.sparsity_lambda_schedule == "delayed_linear":
            assert 0.0 <= self.sparsity_lambda_delay_frac < 1.0, (
                "sparsity_lambda_delay_frac must be between 0.0 (inclusive) and 1.0 (exclusive)"
            )
        assert self.normalization_method in NORM_METHODS, (
            f"Invalid normalization_method: {self.normalization_method}. Must be one of {list(NORM_METHODS)}"
        )
        assert self.optimizer in ("adam", "adamw"), f"Invalid optimizer: {self.optimizer}"
        assert self.lr_scheduler in (None, "linear", "cosine", "linear_final20"), (
            f"Invalid lr_scheduler: {self.lr_scheduler}"
        )
        assert self.engine in ("auto", "fused", "autograd"), f"Invalid engine: {self.engine}"

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


@dataclass
class InferenceConfig:
    """Evaluation-run description (reference: clt_config.py:272-311; no consumer there either)."""

    clt_checkpoint_path: str
    data_path: str
    eval_batch_size_tokens: int = 4096
    max_eval_batches: Optional[int] = None
    device: Optional[str] = None
    output_log_dir: str = "clt_inference_results"
    data_source_type: str = "local_manifest"
    generation_config_path: Optional[str] = None
    dataset_params_path: Optional[str] = None
    remote_server_config_path: Optional[str] = None
    activation_dtype: Optional[str] = "float16"
    normalization_method: str = "loaded_mean_std"
    enable_wandb: bool = False
    wandb_project: Optional[str] = "clt_evaluation"
    wandb_entity: Optional[str] = None
    wandb_run_name: Optional[str] = None
    wandb_tags: Optional[List[str]] = field(default_factory=list)
    model_name_for_wandb: Optional[str] = None
    model_world_size_for_load: int = 1
