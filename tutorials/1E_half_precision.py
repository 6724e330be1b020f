#!/usr/bin/env python
"""Tutorial 1E/1G - bf16 and fp16 training (reference: tutorials 1E and 1G, README.md:291-304).

bf16: weights in bf16, fp32 Adam moments, optional stochastic rounding; on a B200 this is the fused step.
fp16: autocast + loss scaling on the autograd step (GPU only).

    python tutorials/1E_half_precision.py
"""
import os

import torch

from _common import clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200.training.trainer import CLTTrainer


def main() -> None:
    root = workdir("1E")
    data = dataset(os.path.join(root, "activations"))
    if not torch.cuda.is_available():
        print("no GPU: running the fp32 configuration; precision='bf16' / 'fp16' need CUDA")
        CLTTrainer(clt_config(), training_config(data, steps=20), log_dir=os.path.join(root, "fp32"), device="cpu").train()
        return
    for precision, extra in (("bf16", dict(enable_stochastic_rounding=True)), ("fp16", {})):
        cfg = clt_config(clt_dtype="bfloat16" if precision == "bf16" else None)
        tc = training_config(data, steps=40, precision=precision, **extra)
        trainer = CLTTrainer(cfg, tc, log_dir=os.path.join(root, precision), device=device())
        print(precision, "engine:", "fused" if trainer.engine is not None else "autograd")
        trainer.train()


if __name__ == "__main__":
    main()
