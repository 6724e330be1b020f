#!/usr/bin/env python
"""Tutorial 1F - tied decoders (per_source / per_target), feature offset / scale and the skip connection
(reference: tutorials/1F-end-to-end-training-gpt2-tied-decoders.py).

    python tutorials/1F_tied_decoders.py
"""
import os

from _common import clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200.training.trainer import CLTTrainer


def main() -> None:
    root = workdir("1F")
    data = dataset(os.path.join(root, "activations"))
    for tying in ("per_source", "per_target"):
        cfg = clt_config(decoder_tying=tying, enable_feature_offset=True, enable_feature_scale=True, skip_connection=True)
        trainer = CLTTrainer(cfg, training_config(data, steps=40), log_dir=os.path.join(root, tying), device=device())
        model = trainer.train()
        n_dec = sum(p.numel() for n, p in model.named_parameters() if "dec" in n)
        print(f"{tying}: decoder parameters {n_dec:,} (untied would be {cfg.num_features * cfg.d_model * cfg.num_layers * (cfg.num_layers + 1) // 2:,})")


if __name__ == "__main__":
    main()
