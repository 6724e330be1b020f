"""The tutorial scripts run end to end on a CPU (they are the user-level API surface: generate -> train -> save /
load -> convert, the server protocol by hand, remote training against a server subprocess)."""
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.integration


def _run(name, tmp_path, *args, expect=0):
    env = dict(os.environ, CLT_TUTORIAL_DIR=str(tmp_path), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run([sys.executable, os.path.join(REPO, "tutorials", name), *args], capture_output=True, text=True, timeout=900,
                         env=env, cwd=os.path.join(REPO, "tutorials"))
    assert res.returncode == expect, res.stdout[-2000:] + res.stderr[-3000:]
    return res.stdout


def test_end_to_end_and_conversion(tmp_path):
    out = _run("1A_end_to_end_batchtopk.py", tmp_path)
    assert "reloaded model" in out
    out = _run("1B_theta_conversion.py", tmp_path)
    assert "activation function is now: jumprelu" in out


def test_topk_and_jumprelu_walkthroughs(tmp_path):
    out = _run("1C_end_to_end_topk.py", tmp_path)
    assert "topk_k=16.0: active features per token min/max = 16/16" in out and "reloaded: topk" in out
    out = _run("1D_end_to_end_jumprelu.py", tmp_path)
    assert "reloaded model with trained thresholds" in out


def test_server_protocol_and_remote_training(tmp_path):
    import socket
    import time

    import requests

    out = _run("3_server_upload_and_slice.py", tmp_path)
    assert "slice: (4, 2, 4, 64)" in out
    out = _run("2_remote_training.py", tmp_path)
    assert "server info" in out
    # tutorial 4 trains from a server somebody else started: none there -> exit code 2, then one serving tutorial 2's data
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    url = f"http://127.0.0.1:{port}"
    assert "no activation server" in _run("4_train_against_running_server.py", tmp_path, "--server-url", url, expect=2)
    env = dict(os.environ, HOST="127.0.0.1", PORT=str(port), STORAGE_BASE_DIR=str(tmp_path / "2" / "server_data"), PYTHONPATH=REPO)
    server = subprocess.Popen([sys.executable, "-m", "crosslayer_coding_b200.server.main"], env=env,
                              stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    try:
        for _ in range(200):
            try:
                if requests.get(url + "/api/v1/health", timeout=1).ok:
                    break
            except requests.RequestException:
                time.sleep(0.1)
        out = _run("4_train_against_running_server.py", tmp_path, "--server-url", url, "--steps", "10")
        assert "trained from the remote store" in out
        assert "is not on the server" in _run("4_train_against_running_server.py", tmp_path, "--server-url", url,
                                              "--dataset-id", "nobody/nothing", expect=3)
    finally:
        server.terminate()
        server.wait(timeout=10)


def test_analysis_helpers(tmp_path):
    import json

    import torch
    from safetensors.torch import save_file

    ck = str(tmp_path / "m.safetensors")
    save_file({"a.weight": torch.randn(4, 3), "b.bias": torch.zeros(5)}, ck)
    res = subprocess.run([sys.executable, os.path.join(REPO, "scripts", "analysis", "check_model.py"), ck], capture_output=True, text=True)
    assert res.returncode == 0 and "all zero" in res.stdout and "17 parameters" in res.stdout
    shard = tmp_path / "top"
    shard.mkdir()
    json.dump({"features": {"3": [{"activation": 1.5, "tokens": ["a", "b"], "activations": [0.1, 1.5]}]}}, open(shard / "s0.json", "w"))
    out = str(tmp_path / "top.html")
    res = subprocess.run([sys.executable, os.path.join(REPO, "scripts", "analysis", "visualize_top_activations.py"),
                          "--input-dir", str(shard), "--output", out], capture_output=True, text=True)
    assert res.returncode == 0 and "feature 3" in open(out).read()
