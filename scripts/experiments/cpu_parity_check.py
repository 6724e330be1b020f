#!/usr/bin/env python
"""Step-by-step parity of the autograd step against the reference implementation on a CPU, in fp32.

Both models start from the same weights (the reference's state dict is loaded into this framework's model through
the reference key names), see the same synthetic batches and take the same AdamW steps; the script prints the
largest relative difference of the loss terms over the run, the final normalised MSE of both, and tokens/s.

    python scripts/experiments/cpu_parity_check.py --reference-root baseline/_ref --steps 200
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=str(REPO / "baseline" / "_ref"))
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--d-model", type=int, default=128)
    ap.add_argument("--features", type=int, default=1024)
    ap.add_argument("--k", type=int, default=32)
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--activation", default="batchtopk", choices=["batchtopk", "jumprelu", "relu", "topk"])
    args = ap.parse_args()
    sys.path.insert(0, args.reference_root)
    try:
        from clt.config import CLTConfig as RefCLTConfig, TrainingConfig as RefTrainingConfig
        from clt.models.clt import CrossLayerTranscoder as RefCLT
        from clt.training.losses import LossManager as RefLossManager
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"unavailable": f"reference import failed: {type(exc).__name__}: {exc}"}))
        return 0
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.activation_generation.synthetic import SparseDictionarySynth, SyntheticSpec
    from crosslayer_coding_b200.training.losses import LossManager

    L, d, F, B = args.layers, args.d_model, args.features, args.batch
    common = dict(num_features=F, num_layers=L, d_model=d, activation_fn=args.activation, batchtopk_k=args.k, topk_k=args.k,
                  jumprelu_threshold=0.03)
    tkw = dict(learning_rate=1e-3, training_steps=args.steps, train_batch_size_tokens=B, activation_path="unused",
               normalization_method="none", sparsity_lambda=1e-3, sparsity_c=1.0, preactivation_coef=3e-6, aux_loss_factor=None,
               apply_sparsity_penalty_to_batchtopk=True, optimizer="adamw", lr_scheduler=None)
    torch.manual_seed(0)
    ref = RefCLT(RefCLTConfig(**common), process_group=None, device=torch.device("cpu"))
    ours = CrossLayerTranscoder(CLTConfig(**common), device="cpu")
    ours.load_state_dict(ref.state_dict())
    ref_loss = RefLossManager(RefTrainingConfig(**tkw))
    our_loss = LossManager(TrainingConfig(**tkw), clt_config=CLTConfig(**common))
    opt_r = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    opt_o = torch.optim.AdamW(ours.parameters(), lr=1e-3)
    synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=4 * d, active_mean=8.0, seed=7), device="cpu")
    synth.fit_norm_stats(4096)
    worst = {}
    t_ref = t_our = 0.0
    for step in range(args.steps):
        x, y = synth.sample(B, seed=100 + step, normalize=True, dtype=torch.float32)
        inputs = {l: x[l] for l in range(L)}
        targets = {l: y[l] for l in range(L)}
        t0 = time.perf_counter()
        opt_r.zero_grad(set_to_none=True)
        lr_, dr = ref_loss.compute_total_loss(ref, inputs, targets, step, args.steps)
        lr_.backward()
        opt_r.step()
        if hasattr(ref, "decoder_module") and hasattr(ref.decoder_module, "_cached_decoder_norms"):
            ref.decoder_module._cached_decoder_norms = None
        t1 = time.perf_counter()
        opt_o.zero_grad(set_to_none=True)
        lo, do = our_loss.compute_total_loss(ours, inputs, targets, step, args.steps)
        lo.backward()
        opt_o.step()
        ours.invalidate_decoder_norms()
        t2 = time.perf_counter()
        t_ref += t1 - t0
        t_our += t2 - t1
        scale = max(max(abs(float(v)) for v in dr.values()), 1e-12)
        for key in ("total", "reconstruction", "sparsity", "preactivation"):
            a, b = float(dr.get(key, 0.0)), float(do.get(key, 0.0))
            # the total can cross zero (BatchTopK keeps negative values, so the tanh penalty can be negative):
            # every term is compared on the scale of the step's largest reference term
            rel = abs(a - b) / scale
            worst[key] = max(worst.get(key, 0.0), rel)
    x, y = synth.sample(B, seed=99999, normalize=True, dtype=torch.float32)
    inputs = {l: x[l] for l in range(L)}
    with torch.no_grad():
        out_r, out_o = ref(inputs), ours(inputs)

    def nmse(out):
        return float(sum(((out[l] - y[l]) ** 2).mean() / y[l].var(dim=0, unbiased=False).mean() for l in range(L)) / L)

    print(json.dumps({
        "config": {**common, "batch": B, "steps": args.steps}, "max_loss_difference_over_largest_term": worst,
        "nmse_heldout": {"reference": nmse(out_r), "ours": nmse(out_o)},
        "tokens_per_s": {"reference": B * args.steps / t_ref, "ours_autograd_cpu": B * args.steps / t_our},
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
