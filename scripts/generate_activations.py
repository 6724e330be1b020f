#!/usr/bin/env python
"""Generate an activation dataset from a Hugging Face model and dataset (reference: scripts/generate_activations.py:15-269).

    python scripts/generate_activations.py --model-name gpt2 --mlp-input-template "transformer.h.{}.mlp" \
        --mlp-output-template "transformer.h.{}.mlp" --dataset-path monology/pile-uncopyrighted \
        --target-total-tokens 2000000 --activation-dir ./activations --storage-type local

``--synthetic L,d,dict`` writes the seeded sparse-dictionary dataset instead (no model, no network).
"""
from __future__ import annotations

import argparse
import logging
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from crosslayer_coding_b200.config import ActivationConfig  # noqa: E402


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Generate CLT training activations", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    p.add_argument("--model-name", required=True)
    p.add_argument("--mlp-input-template", default=None)
    p.add_argument("--mlp-output-template", default=None)
    p.add_argument("--model-dtype", default=None)
    p.add_argument("--dataset-path", default="synthetic")
    p.add_argument("--dataset-split", default="train")
    p.add_argument("--dataset-text-column", default="text")
    p.add_argument("--context-size", type=int, default=128)
    p.add_argument("--inference-batch-size", type=int, default=512)
    p.add_argument("--exclude-special-tokens", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--prepend-bos", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--streaming", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--trust-remote-code", "--dataset-trust-remote-code", dest="trust_remote_code", action=argparse.BooleanOptionalAction, default=False,
                   help="allow custom code of the Hugging Face dataset")
    p.add_argument("--cache_path", "--cache-path", dest="cache_path", default=None, help="Hugging Face dataset cache directory")
    p.add_argument("--max_samples", "--max-samples", dest="max_samples", type=int, default=None, help="stop after this many dataset samples")
    p.add_argument("--target-total-tokens", type=int, default=None)
    p.add_argument("--activation-dir", default="./activations")
    p.add_argument("--output-format", choices=["hdf5", "npz"], default="hdf5")
    p.add_argument("--compression", default="gzip", help="gzip, lz4 (stored uncompressed) or none")
    p.add_argument("--chunk-token-threshold", type=int, default=1_000_000)
    p.add_argument("--activation-dtype", choices=["bfloat16", "float16", "float32"], default="bfloat16")
    p.add_argument("--compute-norm-stats", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--remote-server-url", default=None)
    p.add_argument("--delete-after-upload", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--upload-max-retries", type=int, default=5, help="attempts per chunk upload")
    p.add_argument("--upload-initial-backoff", type=float, default=1.0, help="seconds before the first retry")
    p.add_argument("--upload-max-backoff", type=float, default=30.0, help="cap of the exponential backoff, seconds")
    p.add_argument("--nnsight-tracer-kwargs-json", default="{}", help="JSON dict kept in ActivationConfig.nnsight_tracer_kwargs "
                   "(the extractor uses forward hooks; the field is carried for configuration parity)")
    p.add_argument("--nnsight-invoker-args-json", default="{}", help="JSON dict kept in ActivationConfig.nnsight_invoker_args")
    p.add_argument("--storage-type", choices=["local", "remote"], default="local")
    p.add_argument("--device", default=None)
    p.add_argument("--enable-profiling", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--synthetic", default=None, help="num_layers,d_model,dict_size[,active_mean]: write the synthetic dataset")
    p.add_argument("--seed", type=int, default=0)
    return p


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(levelname)s %(message)s")
    args = build_parser().parse_args(argv)
    compression = None if str(args.compression).lower() in ("none", "false", "") else args.compression
    if args.synthetic:
        import os

        from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset

        parts = [float(v) for v in args.synthetic.split(",")]
        spec = SyntheticSpec(num_layers=int(parts[0]), d_model=int(parts[1]), dict_size=int(parts[2]),
                             active_mean=parts[3] if len(parts) > 3 else 32.0, seed=args.seed)
        out = os.path.join(args.activation_dir, args.model_name, f"{os.path.basename(args.dataset_path)}_{args.dataset_split}")
        write_synthetic_dataset(out, spec, total_tokens=args.target_total_tokens or 1_000_000, chunk_tokens=args.chunk_token_threshold,
                                dtype=args.activation_dtype, device=args.device or "cpu", compression=compression, model_name=args.model_name)
        print(out)
        return 0
    if not args.mlp_input_template or not args.mlp_output_template:
        raise SystemExit("--mlp-input-template and --mlp-output-template are required")
    import json

    try:
        tracer_kwargs = json.loads(args.nnsight_tracer_kwargs_json)
        invoker_args = json.loads(args.nnsight_invoker_args_json)
    except json.JSONDecodeError as exc:
        raise SystemExit(f"--nnsight-*-json must be valid JSON (or '{{}}'): {exc}")
    cfg = ActivationConfig(
        model_name=args.model_name, mlp_input_module_path_template=args.mlp_input_template,
        mlp_output_module_path_template=args.mlp_output_template, dataset_path=args.dataset_path, model_dtype=args.model_dtype,
        activation_dtype=args.activation_dtype, dataset_split=args.dataset_split, dataset_text_column=args.dataset_text_column,
        context_size=args.context_size, inference_batch_size=args.inference_batch_size,
        exclude_special_tokens=args.exclude_special_tokens, prepend_bos=args.prepend_bos, streaming=args.streaming,
        dataset_trust_remote_code=args.trust_remote_code, cache_path=args.cache_path,
        target_total_tokens=args.target_total_tokens, activation_dir=args.activation_dir, output_format=args.output_format,
        compression=compression, chunk_token_threshold=args.chunk_token_threshold, compute_norm_stats=args.compute_norm_stats,
        remote_server_url=args.remote_server_url, delete_after_upload=args.delete_after_upload, enable_profiling=args.enable_profiling,
        upload_max_retries=args.upload_max_retries, upload_initial_backoff=args.upload_initial_backoff,
        upload_max_backoff=args.upload_max_backoff, nnsight_tracer_kwargs=tracer_kwargs, nnsight_invoker_args=invoker_args,
    )
    from crosslayer_coding_b200.activation_generation import ActivationGenerator

    gen = ActivationGenerator(cfg, device=args.device)
    if args.max_samples is not None:
        gen.max_samples = int(args.max_samples)
    gen.set_storage_type(args.storage_type)
    gen.generate_and_save()
    print(gen.out_dir)
    return 0


if __name__ == "__main__":
    sys.exit(main())
