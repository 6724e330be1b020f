#!/usr/bin/env python
"""40-step BatchTopK smoke run on a synthetic pythia-70m-shaped dataset (reference: scripts/smoke_train.py,
scripts/smoke_train_dist.sh).  Single process by default; ``torchrun --nproc_per_node 2 scripts/smoke_train.py``
runs it tensor-parallel.  No network: the dataset is generated locally on first use.
"""
from __future__ import annotations

import logging
import os
import sys
import tempfile
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from crosslayer_coding_b200 import CLTConfig, TrainingConfig  # noqa: E402
from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset  # noqa: E402
from crosslayer_coding_b200.training.trainer import CLTTrainer  # noqa: E402


def main() -> int:
    logging.basicConfig(level=logging.INFO)
    distributed = int(os.environ.get("WORLD_SIZE", "1")) > 1
    rank = int(os.environ.get("RANK", "0"))
    root = os.environ.get("CLT_SMOKE_DIR", os.path.join(tempfile.gettempdir(), "clt_smoke"))
    data = os.path.join(root, "pythia-70m-shaped")
    L, d = 6, 512
    if rank == 0 and not os.path.exists(os.path.join(data, "metadata.json")):
        write_synthetic_dataset(data, SyntheticSpec(num_layers=L, d_model=d, dict_size=2048, active_mean=24, seed=0),
                                total_tokens=int(os.environ.get("CLT_SMOKE_TOKENS", str(64 * 1024))), chunk_tokens=16 * 1024, dtype="bfloat16",
                                device="cuda" if torch.cuda.is_available() else "cpu")
    if distributed:
        import torch.distributed as dist

        if not dist.is_initialized():
            if torch.cuda.is_available():
                local = int(os.environ.get("LOCAL_RANK", "0"))
                torch.cuda.set_device(local)  # before the first collective: one device per rank
                dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
            else:
                dist.init_process_group("gloo")
        dist.barrier()
    on_gpu = torch.cuda.is_available()
    clt = CLTConfig(num_features=4096, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=200,
                    clt_dtype="bfloat16" if on_gpu else None, model_name="pythia-70m-shaped")
    steps = int(os.environ.get("CLT_SMOKE_STEPS", "40"))
    tc = TrainingConfig(learning_rate=1e-4, training_steps=steps, train_batch_size_tokens=1024, activation_path=data,
                        activation_dtype="bfloat16" if on_gpu else "float32", normalization_method="auto",
                        precision="bf16" if on_gpu else "fp32", sparsity_lambda=0.0, preactivation_coef=0.0,
                        apply_sparsity_penalty_to_batchtopk=False, aux_loss_factor=1 / 32, log_interval=10, eval_interval=max(1, steps // 2),
                        checkpoint_interval=max(1, steps // 2), lr_scheduler="linear_final20", optimizer_beta2=0.98)
    trainer = CLTTrainer(clt, tc, log_dir=os.path.join(root, "run"), distributed=distributed)
    trainer.train()
    return 0


if __name__ == "__main__":
    sys.exit(main())
