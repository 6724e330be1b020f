#!/usr/bin/env python
"""Sweep of the AuxK loss factor {1/64 ... 1/512} on a BatchTopK run (reference: scripts/experiments/*: aux-loss sweep
with lr 1e-4, batch 1024, linear_final20, beta2 0.98, k 200-500).  Point ``--activation-path`` at a generated dataset.

    python scripts/experiments/aux_loss_factor_sweep.py --activation-path /data/acts/model/dataset_train --output-dir runs/aux
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from crosslayer_coding_b200 import CLTConfig, TrainingConfig  # noqa: E402
from crosslayer_coding_b200.io.manifest import load_metadata  # noqa: E402
from crosslayer_coding_b200.training.trainer import CLTTrainer  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--activation-path", required=True)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--num-features", type=int, default=16384)
    ap.add_argument("--batchtopk-k", type=int, default=200)
    ap.add_argument("--training-steps", type=int, default=2000)
    ap.add_argument("--train-batch-size-tokens", type=int, default=1024)
    ap.add_argument("--factors", type=float, nargs="+", default=[1 / 64, 1 / 128, 1 / 256, 1 / 512])
    ap.add_argument("--precision", default="bf16")
    ap.add_argument("--device", default=None)
    args = ap.parse_args()
    meta = load_metadata(args.activation_path)
    results = {}
    for factor in args.factors:
        name = f"aux_{factor:.6f}"
        cfg = CLTConfig(num_features=args.num_features, num_layers=int(meta["num_layers"]), d_model=int(meta["d_model"]),
                        activation_fn="batchtopk", batchtopk_k=args.batchtopk_k,
                        clt_dtype="bfloat16" if args.precision == "bf16" else None, model_name=meta.get("model_name", "model"))
        tc = TrainingConfig(learning_rate=1e-4, training_steps=args.training_steps, train_batch_size_tokens=args.train_batch_size_tokens,
                            activation_source="local_manifest", activation_path=args.activation_path, normalization_method="auto",
                            precision=args.precision, sparsity_lambda=0.0, preactivation_coef=0.0, apply_sparsity_penalty_to_batchtopk=False,
                            aux_loss_factor=factor, lr_scheduler="linear_final20", optimizer_beta2=0.98, dead_feature_window=200,
                            eval_interval=max(1, args.training_steps // 4), checkpoint_interval=args.training_steps)
        trainer = CLTTrainer(cfg, tc, log_dir=os.path.join(args.output_dir, name), device=args.device)
        trainer.train()
        metrics = json.load(open(os.path.join(args.output_dir, name, "metrics.json")))
        results[name] = metrics["eval_metrics"][-1] if metrics.get("eval_metrics") else {}
    print(json.dumps(results, indent=1, default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
