#!/usr/bin/env python
"""Generate (or reuse) an activation dataset and run a short BatchTopK training on it, in fp32, bf16 or fp16
(reference: scripts/experiments/run_pythia_batchtopk_training.py and run_pythia_batchtopk_training_fp16.py:
pythia-70m, 32x expansion, k = 200, lr 1e-4, batch 1024, ``linear_final20``, beta2 0.98, AuxK factor 1/32,
no normalisation, float16 activations, fp16 with ``fp16_convert_weights``).

With ``--model-name`` the activations come from that Hugging Face model through forward hooks (the model and the
dataset must be available locally); with ``--synthetic`` (the default) from the seeded sparse-dictionary generator
with the same six layers and width 512, so the run needs no network.

    python scripts/experiments/run_batchtopk_training.py --precision fp16 --training-steps 100
    python scripts/experiments/run_batchtopk_training.py --model-name EleutherAI/pythia-70m \
        --dataset-path monology/pile-uncopyrighted --precision bf16
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from crosslayer_coding_b200 import CLTConfig, TrainingConfig  # noqa: E402
from crosslayer_coding_b200.config.data_config import ActivationConfig  # noqa: E402
from crosslayer_coding_b200.io.manifest import load_metadata  # noqa: E402
from crosslayer_coding_b200.training.trainer import CLTTrainer  # noqa: E402


def ensure_dataset(args) -> str:
    if args.model_name:
        from crosslayer_coding_b200.activation_generation.generator import ActivationGenerator, dataset_id_for

        cfg = ActivationConfig(model_name=args.model_name, mlp_input_module_path_template=args.mlp_input_template,
                               mlp_output_module_path_template=args.mlp_output_template, dataset_path=args.dataset_path,
                               dataset_split="train", dataset_text_column="text", context_size=128, inference_batch_size=192,
                               exclude_special_tokens=True, prepend_bos=True, streaming=True, target_total_tokens=args.tokens,
                               activation_dir=args.activation_dir, output_format="hdf5", compression="gzip",
                               chunk_token_threshold=args.chunk_tokens, activation_dtype=args.activation_dtype, compute_norm_stats=True)
        path = os.path.join(args.activation_dir, dataset_id_for(cfg))
        if not (os.path.exists(os.path.join(path, "metadata.json")) and os.path.exists(os.path.join(path, "index.bin"))):
            t0 = time.time()
            ActivationGenerator(cfg, device=args.device).generate_and_save()
            print(f"generated activations in {time.time() - t0:.1f} s")
        return path
    from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset

    path = os.path.join(args.activation_dir, "synthetic", "pythia70m_shape_train")
    if not os.path.exists(os.path.join(path, "metadata.json")):
        spec = SyntheticSpec(num_layers=args.num_layers, d_model=args.d_model, dict_size=4 * args.d_model, active_mean=16.0, seed=0)
        write_synthetic_dataset(path, spec, total_tokens=args.tokens, chunk_tokens=args.chunk_tokens, dtype=args.activation_dtype,
                                device="cpu")
    return path


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-name", default=None)
    ap.add_argument("--mlp-input-template", default="gpt_neox.layers.{}.mlp.input")
    ap.add_argument("--mlp-output-template", default="gpt_neox.layers.{}.mlp.output")
    ap.add_argument("--dataset-path", default="monology/pile-uncopyrighted")
    ap.add_argument("--synthetic", action="store_true", help="ignored when --model-name is given; the default otherwise")
    ap.add_argument("--num-layers", type=int, default=6)
    ap.add_argument("--d-model", type=int, default=512)
    ap.add_argument("--expansion-factor", type=int, default=32)
    ap.add_argument("--batchtopk-k", type=int, default=200)
    ap.add_argument("--tokens", type=int, default=100_000)
    ap.add_argument("--chunk-tokens", type=int, default=8_000)
    ap.add_argument("--activation-dtype", default="float16", choices=["float16", "bfloat16", "float32"])
    ap.add_argument("--activation-dir", default="./activations_local_100k")
    ap.add_argument("--precision", default="fp32", choices=["fp32", "bf16", "fp16"])
    ap.add_argument("--training-steps", type=int, default=100)
    ap.add_argument("--train-batch-size-tokens", type=int, default=1024)
    ap.add_argument("--learning-rate", type=float, default=1e-4)
    ap.add_argument("--aux-loss-factor", type=float, default=1 / 32)
    ap.add_argument("--output-dir", default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--enable-wandb", action="store_true")
    args = ap.parse_args()
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if args.precision in ("bf16", "fp16") and device == "cpu":
        print(f"precision {args.precision!r} needs a CUDA device; running fp32 on the CPU instead")
        args.precision = "fp32"
    data = ensure_dataset(args)
    meta = load_metadata(data)
    L, d = int(meta["num_layers"]), int(meta["d_model"])
    cfg = CLTConfig(num_features=d * args.expansion_factor, num_layers=L, d_model=d, activation_fn="batchtopk",
                    batchtopk_k=args.batchtopk_k, batchtopk_straight_through=True, model_name=meta.get("model_name", "model"),
                    clt_dtype="bfloat16" if args.precision == "bf16" else None)
    run_name = f"{cfg.num_features}-width-batchtopk-k{args.batchtopk_k}-{args.train_batch_size_tokens}-batch-{args.learning_rate:.1e}-lr"
    tc = TrainingConfig(learning_rate=args.learning_rate, training_steps=args.training_steps, seed=42, activation_source="local_manifest",
                        activation_path=data, activation_dtype=args.activation_dtype, train_batch_size_tokens=args.train_batch_size_tokens,
                        sampling_strategy="sequential", normalization_method="none", sparsity_lambda=0.0, sparsity_lambda_schedule="linear",
                        sparsity_c=0.0, preactivation_coef=0.0, aux_loss_factor=args.aux_loss_factor,
                        apply_sparsity_penalty_to_batchtopk=False, optimizer="adamw", lr_scheduler="linear_final20", optimizer_beta2=0.98,
                        log_interval=10, eval_interval=max(1, args.training_steps // 2), checkpoint_interval=1000, dead_feature_window=1000,
                        enable_wandb=args.enable_wandb, wandb_project="clt-batchtopk", wandb_run_name=run_name,
                        precision=args.precision, fp16_convert_weights=args.precision == "fp16")
    log_dir = args.output_dir or os.path.join("clt_training_logs", f"batchtopk_{args.precision}_{int(time.time())}")
    trainer = CLTTrainer(cfg, tc, log_dir=log_dir, device=device)
    print("run:", run_name, "| engine:", "fused" if getattr(trainer, "engine", None) is not None else "autograd", "| logs:", log_dir)
    t0 = time.time()
    trainer.train()
    dt = time.time() - t0
    metrics = json.load(open(os.path.join(log_dir, "metrics.json")))
    last = metrics["eval_metrics"][-1] if metrics.get("eval_metrics") else {}
    keep = {k: v for k, v in last.items() if isinstance(v, (int, float)) and ("reconstruction/" in k or k in ("sparsity/avg_l0", "step"))}
    print(json.dumps({"seconds": round(dt, 1), "tokens_per_s": round(args.training_steps * args.train_batch_size_tokens / dt, 1), **keep}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
