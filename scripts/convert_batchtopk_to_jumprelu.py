#!/usr/bin/env python
"""Convert a trained BatchTopK / TopK transcoder to JumpReLU (reference: scripts/convert_batchtopk_to_jumprelu.py:90-1053).

Steps: load the model (``.safetensors`` with ``cfg.json`` next to it, a ``.pt`` written by ``model.save``, or a
distributed ``step_N``/``latest`` directory with a merged ``model.safetensors``), estimate per-feature thresholds
over ``--num-batches-for-theta-estimation`` batches, save the converted model and config, report L0 / NMSE / EV
before and after, and with ``--l0-layerwise-calibrate`` scale each layer's thresholds until its L0 matches the
original model's (``crosslayer_coding_b200.conversion``).

    python scripts/convert_batchtopk_to_jumprelu.py --batchtopk-checkpoint-path runs/x/clt_checkpoint_latest.safetensors \
        --config-path runs/x/cfg.json --activation-data-path acts/gpt2/ds_train --output-model-path runs/x/jumprelu.safetensors \
        --output-config-path runs/x/jumprelu_cfg.json --num-batches-for-theta-estimation 50 --l0-layerwise-calibrate
"""
from __future__ import annotations

import argparse
import copy
import json
import logging
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder  # noqa: E402
from crosslayer_coding_b200.conversion import calibrate_layerwise_theta, layer_l0  # noqa: E402
from crosslayer_coding_b200.training.data import LocalActivationStore  # noqa: E402
from crosslayer_coding_b200.training.evaluator import CLTEvaluator  # noqa: E402

logger = logging.getLogger("convert")

# keys written by older training code, mapped to the current names (reference script :33-87)
LEGACY_KEY_MAP = {"encoders.": "encoder_module.encoders.", "decoders.": "decoder_module.decoders.", "log_threshold": "theta_manager.log_threshold"}


def remap_legacy_keys(sd):
    out = {}
    for k, v in sd.items():
        nk = k[len("module."):] if k.startswith("module.") else k
        for old, new in LEGACY_KEY_MAP.items():
            if nk.startswith(old):
                nk = new + nk[len(old):]
                break
        out[nk] = v
    return out


def load_model(checkpoint: str, config_path: str, device) -> CrossLayerTranscoder:
    cfg = CLTConfig.from_json(config_path)
    model = CrossLayerTranscoder(cfg, device=device)
    path = checkpoint
    if os.path.isdir(path):
        path = os.path.join(path, "model.safetensors")
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file

        sd = load_file(path)
    else:
        blob = torch.load(path, map_location="cpu", weights_only=False)
        sd = blob.get("state_dict", blob) if isinstance(blob, dict) else blob
    sd = remap_legacy_keys(sd)
    sd = {k: v for k, v in sd.items() if k != "theta_manager.log_threshold" or cfg.activation_fn == "jumprelu"}
    model.load_state_dict(sd)
    return model


def evaluate(model, store, batches: int, device) -> dict:
    ev = CLTEvaluator(model, device, mean_tg=store.mean_tg, std_tg=store.std_tg,
                      normalization_method=store.normalization_method, d_model=model.config.d_model)
    acc = {}
    n = 0
    for i, (x, y) in enumerate(store):
        if i >= batches:
            break
        m = ev.compute_metrics(x, y)
        for k in ("sparsity/avg_l0", "reconstruction/normalized_mean_reconstruction_error", "reconstruction/explained_variance"):
            acc[k] = acc.get(k, 0.0) + m[k]
        n += 1
    return {k: v / max(1, n) for k, v in acc.items()}


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(levelname)s %(message)s")
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batchtopk-checkpoint-path", required=True)
    ap.add_argument("--config-path", required=True)
    ap.add_argument("--activation-data-path", required=True)
    ap.add_argument("--output-model-path", required=True)
    ap.add_argument("--output-config-path", required=True)
    ap.add_argument("--num-batches-for-theta-estimation", type=int, default=50)
    ap.add_argument("--default-theta-value", type=float, default=1e6)
    ap.add_argument("--batch-size-tokens", type=int, default=4096)
    ap.add_argument("--activation-dtype", default="float32")
    ap.add_argument("--normalization-method", default="auto")
    ap.add_argument("--norm-stats-path", default=None, help="use this norm_stats.json instead of the dataset's")
    ap.add_argument("--eval-batches", type=int, default=4)
    ap.add_argument("--l0-layerwise-calibrate", action="store_true")
    ap.add_argument("--l0-calibration-batches", type=int, default=1)
    ap.add_argument("--l0-calibration-tolerance", type=float, default=0.5)
    ap.add_argument("--device", default=None)
    ap.add_argument("--seed", type=int, default=42)
    args = ap.parse_args(argv)
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = load_model(args.batchtopk_checkpoint_path, args.config_path, device)
    if model.config.activation_fn not in ("batchtopk", "topk"):
        raise SystemExit(f"model activation is {model.config.activation_fn!r}; nothing to convert")

    def make_store():
        st = LocalActivationStore(args.activation_data_path, train_batch_size_tokens=args.batch_size_tokens, device=device,
                                  dtype=args.activation_dtype, normalization_method=args.normalization_method, seed=args.seed,
                                  shard_data=False)
        if args.norm_stats_path:
            with open(args.norm_stats_path) as fh:
                st._prep_norm(json.load(fh))
        return st

    store = make_store()
    before = evaluate(model, store, args.eval_batches, device)
    store.close()
    logger.info("original model: %s", before)
    calib = None
    target_l0 = None
    if args.l0_layerwise_calibrate:
        store = make_store()
        xs = [next(store)[0] for _ in range(args.l0_calibration_batches)]
        calib = {l: torch.cat([x[l] for x in xs]) for l in xs[0]}
        store.close()
        target_l0 = layer_l0(model, calib)
    store = make_store()
    model.estimate_theta_posthoc(store, num_batches=args.num_batches_for_theta_estimation, default_theta_value=args.default_theta_value)
    store.close()
    if calib is not None:
        scales = calibrate_layerwise_theta(model, calib, target_l0, tolerance=args.l0_calibration_tolerance)
        logger.info("layer-wise scales: %s", scales)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_model_path)), exist_ok=True)
    from safetensors.torch import save_file

    save_file({k: v.detach().cpu().clone().contiguous() for k, v in model.state_dict().items()}, args.output_model_path)
    model.config.to_json(args.output_config_path)
    store = make_store()
    after = evaluate(model, store, args.eval_batches, device)
    store.close()
    logger.info("converted model: %s", after)
    print(json.dumps({"before": before, "after": after}, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
