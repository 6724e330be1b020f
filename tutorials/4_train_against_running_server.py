#!/usr/bin/env python
"""Tutorial 4 - train from an activation server that is already running somewhere else
(reference: tutorials/4-remote-server-training-test.py).

Unlike tutorial 2 nothing is started or uploaded here: the script checks ``/api/v1/health``, reads the dataset's
``info`` / ``norm_stats`` / manifest through the client and trains for a few steps from ``POST .../slice`` batches.

    STORAGE_BASE_DIR=/data/server python -m crosslayer_coding_b200.server.main &          # on the serving host
    python tutorials/4_train_against_running_server.py --server-url http://127.0.0.1:8000 --dataset-id synthetic/toy_train
"""
import argparse
import os
import sys

import requests

from _common import clt_config, device, training_config, workdir

from crosslayer_coding_b200.training.trainer import CLTTrainer


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--server-url", default=os.environ.get("CLT_SERVER_URL", "http://127.0.0.1:8000"))
    ap.add_argument("--dataset-id", default=os.environ.get("CLT_DATASET_ID", "synthetic/toy_train"))
    ap.add_argument("--steps", type=int, default=30)
    args = ap.parse_args()
    try:
        ok = requests.get(args.server_url.rstrip("/") + "/api/v1/health", timeout=3).ok
    except requests.RequestException as e:
        print(f"no activation server at {args.server_url}: {type(e).__name__}")
        return 2
    if not ok:
        print("server is up but not healthy")
        return 2
    quoted = requests.utils.quote(args.dataset_id, safe="")
    info = requests.get(f"{args.server_url.rstrip('/')}/datasets/{quoted}/info", timeout=10)
    if info.status_code != 200:
        print(f"dataset {args.dataset_id!r} is not on the server (HTTP {info.status_code})")
        return 3
    meta = info.json()
    print("dataset:", {k: meta[k] for k in ("num_layers", "d_model", "total_tokens") if k in meta})
    cfg = clt_config(num_layers=int(meta["num_layers"]), d_model=int(meta["d_model"]))
    tc = training_config(None, steps=args.steps, activation_source="remote", activation_path=None,
                         remote_config={"server_url": args.server_url, "dataset_id": args.dataset_id, "timeout": 60,
                                        "max_retries": 3, "prefetch_batches": 4})
    CLTTrainer(cfg, tc, log_dir=os.path.join(workdir("4"), "run"), device=device()).train()
    print("trained from the remote store")
    return 0


if __name__ == "__main__":
    sys.exit(main())
