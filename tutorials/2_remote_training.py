#!/usr/bin/env python
"""Tutorial 2 - start the activation server as a subprocess, publish a dataset to it and train from it
(reference: tutorials/2-remote-training.py).  Everything stays on 127.0.0.1.

    python tutorials/2_remote_training.py
"""
import os
import shutil
import socket
import subprocess
import sys
import time

import requests

from _common import REPO, clt_config, dataset, device, training_config, workdir

from crosslayer_coding_b200.training.trainer import CLTTrainer


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main() -> None:
    root = workdir("2")
    data = dataset(os.path.join(root, "activations"))
    # the server serves <STORAGE_BASE_DIR>/<dataset_id>/ ; the dataset id has the form <model>/<dataset>_<split>
    storage = os.path.join(root, "server_data")
    dataset_id = "synthetic/toy_train"
    target = os.path.join(storage, dataset_id)
    if not os.path.exists(target):
        os.makedirs(os.path.dirname(target), exist_ok=True)
        shutil.copytree(data, target)
    port = free_port()
    env = dict(os.environ, HOST="127.0.0.1", PORT=str(port), STORAGE_BASE_DIR=storage, PYTHONPATH=str(REPO))
    server = subprocess.Popen([sys.executable, "-m", "crosslayer_coding_b200.server.main"], env=env,
                              stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    url = f"http://127.0.0.1:{port}"
    try:
        for _ in range(100):
            try:
                if requests.get(url + "/api/v1/health", timeout=1).ok:
                    break
            except requests.RequestException:
                time.sleep(0.1)
        print("server info:", requests.get(f"{url}/datasets/{requests.utils.quote(dataset_id, safe='')}/info", timeout=5).json())
        tc = training_config(data, steps=30, activation_source="remote", activation_path=None,
                             remote_config={"server_url": url, "dataset_id": dataset_id, "timeout": 30, "max_retries": 3})
        CLTTrainer(clt_config(), tc, log_dir=os.path.join(root, "run"), device=device()).train()
    finally:
        server.terminate()
        server.wait(timeout=10)


if __name__ == "__main__":
    main()
