#!/usr/bin/env python
"""Train a cross-layer transcoder from a pre-generated activation dataset (local manifest or remote server).

Command line of the reference trainer script (scripts/train_clt.py:96-491): the same flags map one-to-one onto
``CLTConfig`` / ``TrainingConfig``; ``cli_args.json`` is written into the run directory and re-read on
``--resume_from_checkpoint_dir`` (with ``--training-steps`` as the only override), and the checkpoint picked is
``latest`` / ``step_N`` (distributed) or ``clt_checkpoint_{latest|N}.safetensors`` (single process).

    python scripts/train_clt.py --activation-source local_manifest --activation-path acts/gpt2/ds_train \
        --model-name gpt2 --num-features 24576 --activation-fn batchtopk --batchtopk-k 200 --clt-dtype bfloat16 \
        --precision bf16 --learning-rate 1e-4 --training-steps 50000 --output-dir runs/gpt2_32x
    torchrun --nproc_per_node 8 scripts/train_clt.py --distributed ...

Model dimensions come from the dataset's ``metadata.json`` (or ``--num-layers/--d-model``), falling back to the
Hugging Face config of ``--model-name`` when it is available offline.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from crosslayer_coding_b200 import CLTConfig, TrainingConfig  # noqa: E402

logger = logging.getLogger("train_clt")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Train a Cross-Layer Transcoder", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    g = p.add_argument_group("Core")
    g.add_argument("--activation-source", choices=["local_manifest", "remote"], required=True)
    g.add_argument("--output-dir", default=None, help="run directory (default: clt_train_<timestamp>)")
    g.add_argument("--model-name", required=True, help="base model name (dimension lookup and bookkeeping)")
    g.add_argument("--device", default=None)
    g.add_argument("--distributed", action="store_true", help="tensor-parallel run under torchrun")
    g.add_argument("--resume_from_checkpoint_dir", default=None)
    g.add_argument("--resume_step", type=int, default=None)
    g.add_argument("--num-layers", type=int, default=None)
    g.add_argument("--d-model", type=int, default=None)
    g = p.add_argument_group("Local activation source")
    g.add_argument("--activation-path", default=None)
    g = p.add_argument_group("Remote activation source")
    g.add_argument("--server-url", default=None)
    g.add_argument("--dataset-id", default=None)
    g.add_argument("--remote-timeout", type=int, default=120)
    g.add_argument("--remote-max-retries", type=int, default=3)
    g.add_argument("--remote-prefetch-batches", type=int, default=16)
    g = p.add_argument_group("CLT architecture")
    g.add_argument("--num-features", type=int, required=True)
    g.add_argument("--activation-fn", choices=["jumprelu", "relu", "batchtopk", "topk"], default="jumprelu")
    g.add_argument("--jumprelu-threshold", type=float, default=0.03)
    g.add_argument("--batchtopk-k", type=int, default=None)
    g.add_argument("--batchtopk-frac", type=float, default=None, help="alternative to --batchtopk-k: fraction of L*F")
    g.add_argument("--disable-batchtopk-straight-through", action="store_true")
    g.add_argument("--topk-mode", choices=["global", "per_layer"], default="global")
    g.add_argument("--topk-k", type=float, default=None)
    g.add_argument("--disable-topk-straight-through", action="store_true")
    g.add_argument("--clt-dtype", default=None)
    g.add_argument("--decoder-tying", choices=["none", "per_source", "per_target"], default="none")
    g.add_argument("--enable-feature-offset", action="store_true")
    g.add_argument("--enable-feature-scale", action="store_true")
    g.add_argument("--skip-connection", action="store_true")
    g = p.add_argument_group("Training")
    g.add_argument("--learning-rate", type=float, default=3e-4)
    g.add_argument("--training-steps", type=int, default=50000)
    g.add_argument("--train-batch-size-tokens", type=int, default=4096)
    g.add_argument("--precision", choices=["fp32", "fp16", "bf16"], default="fp32")
    g.add_argument("--fp16-convert-weights", action="store_true")
    g.add_argument("--debug-anomaly", action="store_true")
    g.add_argument("--normalization-method", choices=["none", "mean_std", "sqrt_d_model", "auto"], default="mean_std")
    g.add_argument("--sparsity-lambda", type=float, default=1e-3)
    g.add_argument("--sparsity-lambda-schedule", choices=["linear", "delayed_linear"], default="linear")
    g.add_argument("--sparsity-lambda-delay-frac", type=float, default=0.1)
    g.add_argument("--sparsity-c", type=float, default=1.0)
    g.add_argument("--preactivation-coef", type=float, default=3e-6)
    g.add_argument("--aux-loss-factor", type=float, default=None)
    g.add_argument("--apply-sparsity-penalty-to-batchtopk", action=argparse.BooleanOptionalAction, default=True)
    g.add_argument("--optimizer", choices=["adam", "adamw"], default="adamw")
    g.add_argument("--optimizer-beta1", type=float, default=None)
    g.add_argument("--optimizer-beta2", type=float, default=None)
    g.add_argument("--lr-scheduler", choices=["linear", "cosine", "linear_final20", "none"], default="linear")
    g.add_argument("--gradient-clip-val", type=float, default=None)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--activation-dtype", choices=["bfloat16", "float16", "float32"], default="bfloat16")
    g.add_argument("--dead-feature-window", type=int, default=1000)
    g.add_argument("--compute-sparsity-diagnostics", action="store_true")
    g.add_argument("--enable-profiling", action="store_true")
    g.add_argument("--enable-stochastic-rounding", action="store_true")
    g.add_argument("--engine", choices=["auto", "fused", "autograd"], default="auto")
    g.add_argument("--optimizer-states-dtype", choices=["model_dtype", "float32", "bfloat16"], default="model_dtype",
                   help="fused step: fp32 moments unless 'bfloat16' (stochastically rounded bf16 moments)")
    g.add_argument("--fused-max-active-per-token", type=int, default=1024,
                   help="fused JumpReLU step: capacity of the active-entry lists per token")
    g.add_argument("--peer-health-timeout-s", type=float, default=None,
                   help="tensor-parallel runs: declare a rank lost when it has not announced the next step for this long")
    g.add_argument("--async-checkpoint", action=argparse.BooleanOptionalAction, default=None,
                   help="snapshot the state to pinned memory on a side stream and write checkpoints from a thread (default: on for CUDA runs)")
    g.add_argument("--loss-scale-init", type=float, default=65536.0, help="fp16 on the fused step: initial dynamic loss scale")
    g.add_argument("--loss-scale-growth-interval", type=int, default=2000,
                   help="fp16 on the fused step: steps without overflow before the loss scale doubles")
    g.add_argument("--prefetch-batches", type=int, default=2)
    g.add_argument("--sampling-strategy", choices=["sequential", "random_chunk"], default="sequential")
    g = p.add_argument_group("Logging")
    g.add_argument("--log-interval", type=int, default=100)
    g.add_argument("--eval-interval", type=int, default=1000)
    g.add_argument("--checkpoint-interval", type=int, default=1000)
    g.add_argument("--enable-wandb", action="store_true")
    g.add_argument("--wandb-project", default=None)
    g.add_argument("--wandb-entity", default=None)
    g.add_argument("--wandb-run-name", default=None)
    g.add_argument("--wandb-tags", nargs="*", default=None)
    return p


def model_dimensions(args) -> tuple:
    """(num_layers, d_model): explicit flags, then the dataset metadata, then the HF config."""
    if args.num_layers and args.d_model:
        return args.num_layers, args.d_model
    if args.activation_source == "local_manifest" and args.activation_path:
        meta = Path(args.activation_path) / "metadata.json"
        if meta.exists():
            m = json.loads(meta.read_text())
            return int(m["num_layers"]), int(m["d_model"])
    if args.activation_source == "remote" and args.server_url and args.dataset_id:
        try:
            import requests
            from urllib.parse import quote

            r = requests.get(f"{args.server_url.rstrip('/')}/datasets/{quote(args.dataset_id, safe='')}/info", timeout=args.remote_timeout)
            if r.ok:
                return int(r.json()["num_layers"]), int(r.json()["d_model"])
        except Exception as exc:  # noqa: BLE001
            logger.warning("could not read dataset info from the server: %s", exc)
    try:
        from transformers import AutoConfig

        hf = AutoConfig.from_pretrained(args.model_name)
        layers = getattr(hf, "num_hidden_layers", None) or getattr(hf, "n_layer", None)
        width = getattr(hf, "hidden_size", None) or getattr(hf, "n_embd", None)
        if layers and width:
            return int(layers), int(width)
    except Exception as exc:  # noqa: BLE001
        logger.warning("could not load the Hugging Face config of %s: %s", args.model_name, exc)
    raise SystemExit("cannot determine num_layers / d_model: pass --num-layers and --d-model")


def resolve_resume(args):
    """Returns (args, run_dir, checkpoint_path or None), merging the saved cli_args.json on resume."""
    if not args.resume_from_checkpoint_dir:
        run_dir = args.output_dir or f"clt_train_{int(time.time())}"
        return args, run_dir, None
    base = Path(args.resume_from_checkpoint_dir)
    saved = base / "cli_args.json"
    if saved.exists():
        merged = json.loads(saved.read_text())
        merged.update(resume_from_checkpoint_dir=args.resume_from_checkpoint_dir, resume_step=args.resume_step, output_dir=str(base.resolve()))
        if merged.get("training_steps") != args.training_steps:
            logger.info("overriding training_steps %s -> %s", merged.get("training_steps"), args.training_steps)
            merged["training_steps"] = args.training_steps
        merged["distributed"] = args.distributed or merged.get("distributed", False)
        args = argparse.Namespace(**{**vars(args), **merged})
    else:
        logger.warning("%s not found; using the current command line only", saved)
    if args.distributed:
        ckpt = base / (f"step_{args.resume_step}" if args.resume_step is not None else "latest")
    else:
        ckpt = base / (f"clt_checkpoint_{args.resume_step}.safetensors" if args.resume_step is not None else "clt_checkpoint_latest.safetensors")
    if not ckpt.exists():
        raise SystemExit(f"checkpoint to resume from does not exist: {ckpt}")
    return args, str(base.resolve()), str(ckpt)


def configs_from_args(args):
    num_layers, d_model = model_dimensions(args)
    k = args.batchtopk_k
    if args.activation_fn == "batchtopk" and k is None and args.batchtopk_frac is not None:
        k = max(1, int(args.batchtopk_frac * args.num_features * num_layers))
    clt_config = CLTConfig(
        num_features=args.num_features, num_layers=num_layers, d_model=d_model, model_name=args.model_name,
        normalization_method=args.normalization_method, activation_fn=args.activation_fn,
        jumprelu_threshold=args.jumprelu_threshold, batchtopk_k=k,
        batchtopk_straight_through=not args.disable_batchtopk_straight_through, topk_k=args.topk_k,
        topk_straight_through=not args.disable_topk_straight_through, topk_mode=args.topk_mode, clt_dtype=args.clt_dtype,
        decoder_tying=args.decoder_tying, enable_feature_offset=args.enable_feature_offset,
        enable_feature_scale=args.enable_feature_scale, skip_connection=args.skip_connection,
    )
    remote = None
    if args.activation_source == "remote":
        if not args.server_url or not args.dataset_id:
            raise SystemExit("--server-url and --dataset-id are required with --activation-source remote")
        remote = {"server_url": args.server_url, "dataset_id": args.dataset_id, "timeout": args.remote_timeout,
                  "max_retries": args.remote_max_retries, "prefetch_batches": args.remote_prefetch_batches}
    run_name = args.wandb_run_name
    if args.enable_wandb and not run_name:
        run_name = f"{args.num_features}-width-{args.activation_fn}-{args.train_batch_size_tokens}-batch-{args.learning_rate:.1e}-lr"
    training_config = TrainingConfig(
        learning_rate=args.learning_rate, training_steps=args.training_steps, seed=args.seed,
        gradient_clip_val=args.gradient_clip_val, train_batch_size_tokens=args.train_batch_size_tokens,
        precision=args.precision, fp16_convert_weights=args.fp16_convert_weights, debug_anomaly=args.debug_anomaly,
        normalization_method=args.normalization_method, activation_source=args.activation_source,
        activation_dtype=args.activation_dtype, activation_path=args.activation_path, remote_config=remote,
        sampling_strategy=args.sampling_strategy, sparsity_lambda=args.sparsity_lambda,
        sparsity_lambda_schedule=args.sparsity_lambda_schedule, sparsity_lambda_delay_frac=args.sparsity_lambda_delay_frac,
        sparsity_c=args.sparsity_c, preactivation_coef=args.preactivation_coef, aux_loss_factor=args.aux_loss_factor,
        apply_sparsity_penalty_to_batchtopk=args.apply_sparsity_penalty_to_batchtopk, optimizer=args.optimizer,
        optimizer_beta1=args.optimizer_beta1, optimizer_beta2=args.optimizer_beta2,
        lr_scheduler=None if args.lr_scheduler == "none" else args.lr_scheduler, log_interval=args.log_interval,
        eval_interval=args.eval_interval, checkpoint_interval=args.checkpoint_interval,
        compute_sparsity_diagnostics=args.compute_sparsity_diagnostics, enable_profiling=args.enable_profiling,
        dead_feature_window=args.dead_feature_window, enable_wandb=args.enable_wandb, wandb_project=args.wandb_project,
        wandb_entity=args.wandb_entity, wandb_run_name=run_name, wandb_tags=args.wandb_tags or [],
        enable_stochastic_rounding=getattr(args, "enable_stochastic_rounding", False), engine=getattr(args, "engine", "auto"),
        optimizer_states_dtype=getattr(args, "optimizer_states_dtype", "model_dtype"),
        fused_max_active_per_token=getattr(args, "fused_max_active_per_token", 1024),
        peer_health_timeout_s=getattr(args, "peer_health_timeout_s", None), prefetch_batches=getattr(args, "prefetch_batches", 2),
        async_checkpoint=getattr(args, "async_checkpoint", None), loss_scale_init=getattr(args, "loss_scale_init", 65536.0),
        loss_scale_growth_interval=getattr(args, "loss_scale_growth_interval", 2000),
    )
    return clt_config, training_config


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(levelname)s %(message)s")
    args = build_parser().parse_args(argv)
    args, run_dir, ckpt = resolve_resume(args)
    clt_config, training_config = configs_from_args(args)
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        os.makedirs(run_dir, exist_ok=True)
        if ckpt is None:
            with open(os.path.join(run_dir, "cli_args.json"), "w") as fh:
                json.dump(vars(args), fh, indent=2)
    from crosslayer_coding_b200.training.trainer import CLTTrainer

    trainer = CLTTrainer(clt_config, training_config, log_dir=run_dir, device=args.device, distributed=args.distributed,
                         resume_from_checkpoint_path=ckpt)
    trainer.train()
    logger.info("training finished; run directory: %s", run_dir)
    return 0


if __name__ == "__main__":
    sys.exit(main())
