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
from crosslayer_coding_b200.conversion import calibrate_layerwise_theta, layer_l0, quick_l0_check  # noqa: E402
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


def fetch_inputs(make_store, batches: int):
    """``batches`` input batches of a fresh store, concatenated per layer."""
    store = make_store()
    xs = []
    for _ in range(max(1, batches)):
        try:
            xs.append(next(store)[0])
        except StopIteration:
            break
    store.close()
    if not xs:
        raise SystemExit("the activation store yielded no batch")
    return {l: torch.cat([x[l] for x in xs]) for l in xs[0]}


def log_l0_table(title: str, l0s: dict, target: dict = None) -> None:
    logger.info("%s", title)
    for l in sorted(l0s):
        if target is not None and l in target:
            logger.info("  layer %2d: L0 %8.2f   target %8.2f   diff %+8.2f", l, l0s[l], target[l], l0s[l] - target[l])
        else:
            logger.info("  layer %2d: L0 %8.2f", l, l0s[l])
    finite = [v for v in l0s.values() if v == v]
    logger.info("  total L0 %.2f", sum(finite))


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batchtopk-checkpoint-path", required=True, help="checkpoint of the BatchTopK / TopK model (.safetensors, .pt or a sharded directory)")
    ap.add_argument("--config-path", required=True, help="cfg.json of that model")
    ap.add_argument("--activation-data-path", required=True, help="activation dataset directory (LocalActivationStore)")
    ap.add_argument("--output-model-path", required=True)
    ap.add_argument("--output-config-path", required=True)
    ap.add_argument("--num-batches-for-theta-estimation", type=int, default=100)
    ap.add_argument("--estimation-batch-size-tokens", "--batch-size-tokens", dest="estimation_batch_size_tokens", type=int, default=1024,
                    help="tokens per batch for the threshold estimation")
    ap.add_argument("--default-theta-value", type=float, default=1e6, help="threshold of features that never activated")
    ap.add_argument("--device", default=None)
    ap.add_argument("--activation-dtype", default="float32")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--normalization-method", default="auto")
    # quick empirical L0 check of the converted model (reference :253-393, :766-870)
    ap.add_argument("--num-tokens-for-l0-check-script", type=int, default=1024, help="random tokens sampled for the empirical L0 check")
    ap.add_argument("--num-batches-for-l0-check", type=int, default=1, help="batches fetched for the empirical L0 check")
    ap.add_argument("--l0-check-batch-size-tokens", type=int, default=None, help="defaults to --estimation-batch-size-tokens")
    # layer-wise calibration (reference :519-526, :649-763)
    ap.add_argument("--l0-layerwise-calibrate", action="store_true", help="scale every layer's thresholds until its L0 matches the original model's")
    ap.add_argument("--l0-calibration-batches", type=int, default=1)
    ap.add_argument("--l0-calibration-batch-size-tokens", type=int, default=None, help="defaults to --l0-check-batch-size-tokens, then --estimation-batch-size-tokens")
    ap.add_argument("--l0-target-model-config-path", default=None, help="config of the model that defines the target L0s; defaults to --config-path")
    ap.add_argument("--l0-target-model-checkpoint-path", default=None, help="checkpoint of that model; defaults to --batchtopk-checkpoint-path")
    ap.add_argument("--l0-calibration-tolerance", type=float, default=0.5)
    ap.add_argument("--l0-calibration-search-min-scale", type=float, default=0.1)
    ap.add_argument("--l0-calibration-search-max-scale", type=float, default=10.0)
    ap.add_argument("--l0-calibration-max-iters", type=int, default=15)
    ap.add_argument("--norm-stats-path", default=None, help="use this norm_stats.json instead of the dataset's (the training statistics give consistent NMSE / EV)")
    ap.add_argument("--eval-batches", type=int, default=4, help="batches for the NMSE / EV report before and after")
    return ap


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(levelname)s %(message)s")
    args = build_parser().parse_args(argv)
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    torch.manual_seed(args.seed)
    model = load_model(args.batchtopk_checkpoint_path, args.config_path, device)
    if model.config.activation_fn not in ("batchtopk", "topk"):
        raise SystemExit(f"model activation is {model.config.activation_fn!r}; nothing to convert")
    check_bs = args.l0_check_batch_size_tokens or args.estimation_batch_size_tokens
    calib_bs = args.l0_calibration_batch_size_tokens or check_bs

    def store_factory(batch_tokens: int):
        def make():
            st = LocalActivationStore(args.activation_data_path, train_batch_size_tokens=batch_tokens, device=device,
                                      dtype=args.activation_dtype, normalization_method=args.normalization_method, seed=args.seed,
                                      shard_data=False)
            if args.norm_stats_path:
                with open(args.norm_stats_path) as fh:
                    st._prep_norm(json.load(fh))
            return st
        return make

    make_store = store_factory(args.estimation_batch_size_tokens)
    store = make_store()
    before = evaluate(model, store, args.eval_batches, device)
    store.close()
    logger.info("original model: %s", before)

    # targets of the calibration come from the original model, or from a separate one when asked for
    calib = None
    target_l0 = None
    if args.l0_layerwise_calibrate:
        calib = fetch_inputs(store_factory(calib_bs), args.l0_calibration_batches)
        if args.l0_target_model_checkpoint_path or args.l0_target_model_config_path:
            target_model = load_model(args.l0_target_model_checkpoint_path or args.batchtopk_checkpoint_path,
                                      args.l0_target_model_config_path or args.config_path, device)
        else:
            target_model = model
        target_l0 = quick_l0_check(target_model, calib, num_tokens=args.num_tokens_for_l0_check_script, seed=args.seed) \
            if target_model.config.activation_fn not in ("batchtopk", "topk") else layer_l0(target_model, calib)
        log_l0_table("target L0 per layer (original model on the calibration tokens)", target_l0)
        if target_model is not model:
            del target_model

    store = make_store()
    model.estimate_theta_posthoc(store, num_batches=args.num_batches_for_theta_estimation, default_theta_value=args.default_theta_value)
    store.close()
    os.makedirs(os.path.dirname(os.path.abspath(args.output_model_path)), exist_ok=True)
    from safetensors.torch import save_file

    def save():
        save_file({k: v.detach().cpu().clone().contiguous() for k, v in model.state_dict().items()}, args.output_model_path)
        model.config.to_json(args.output_config_path)

    save()
    # empirical L0 of the converted model on freshly fetched tokens
    check_inputs = fetch_inputs(store_factory(check_bs), args.num_batches_for_l0_check)
    l0_converted = quick_l0_check(model, check_inputs, num_tokens=args.num_tokens_for_l0_check_script, seed=args.seed)
    log_l0_table("empirical L0 of the converted model", l0_converted, target_l0)
    report = {"before": before, "l0_converted": l0_converted}
    if calib is not None:
        scales = calibrate_layerwise_theta(
            model, calib, target_l0, tolerance=args.l0_calibration_tolerance,
            scale_range=(args.l0_calibration_search_min_scale, args.l0_calibration_search_max_scale),
            refine_steps=args.l0_calibration_max_iters, seed=args.seed)
        logger.info("layer-wise scales: %s", scales)
        save()  # the calibrated thresholds replace the first save
        l0_calibrated = quick_l0_check(model, check_inputs, num_tokens=args.num_tokens_for_l0_check_script, seed=args.seed)
        log_l0_table("empirical L0 after layer-wise calibration", l0_calibrated, target_l0)
        report.update(target_l0=target_l0, scales=scales, l0_calibrated=l0_calibrated)
    store = make_store()
    after = evaluate(model, store, args.eval_batches, device)
    store.close()
    logger.info("converted model: %s", after)
    report["after"] = after
    print(json.dumps(report, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
