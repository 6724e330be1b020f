"""The command-line tools, end to end on a tiny synthetic dataset (CPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.integration


def _run(script, *args):
    res = subprocess.run([sys.executable, os.path.join(REPO, "scripts", script), *args], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    return res.stdout


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    root = tmp_path_factory.mktemp("cli")
    out = _run("generate_activations.py", "--model-name", "toy", "--dataset-path", "syn", "--synthetic", "2,8,24,4",
               "--target-total-tokens", "512", "--chunk-token-threshold", "128", "--activation-dtype", "float32",
               "--activation-dir", str(root / "acts"), "--compression", "none")
    data = out.strip().splitlines()[-1]
    assert os.path.exists(os.path.join(data, "index.bin"))
    return root, data


def test_train_resume_convert_pipeline(workdir):
    root, data = workdir
    run = str(root / "run")
    common = ["--activation-source", "local_manifest", "--activation-path", data, "--model-name", "toy", "--num-features", "32",
              "--activation-fn", "batchtopk", "--batchtopk-k", "4", "--train-batch-size-tokens", "32", "--activation-dtype", "float32",
              "--learning-rate", "1e-2", "--eval-interval", "5", "--checkpoint-interval", "5", "--log-interval", "2",
              "--sparsity-lambda", "0", "--preactivation-coef", "0", "--device", "cpu"]
    _run("train_clt.py", *common, "--training-steps", "6", "--output-dir", run)
    assert os.path.exists(os.path.join(run, "cli_args.json")) and os.path.exists(os.path.join(run, "clt_checkpoint_5.safetensors"))
    _run("train_clt.py", *common, "--training-steps", "9", "--resume_from_checkpoint_dir", run)
    metrics = json.load(open(os.path.join(run, "metrics.json")))
    assert metrics["train_losses"][-1]["step"] == 8
    out = _run("convert_batchtopk_to_jumprelu.py", "--batchtopk-checkpoint-path", os.path.join(run, "clt_checkpoint_latest.safetensors"),
               "--config-path", os.path.join(run, "cfg.json"), "--activation-data-path", data, "--output-model-path", str(root / "jr.safetensors"),
               "--output-config-path", str(root / "jr.json"), "--num-batches-for-theta-estimation", "4", "--batch-size-tokens", "64",
               "--l0-layerwise-calibrate", "--eval-batches", "2", "--device", "cpu")
    report = json.loads(out[out.index("{"):])
    assert json.load(open(root / "jr.json"))["activation_fn"] == "jumprelu"
    assert abs(report["after"]["sparsity/avg_l0"] - report["before"]["sparsity/avg_l0"]) < 2.0
    _run("analysis/collect_top_activations.py", "--checkpoint", str(root / "jr.safetensors"), "--config", str(root / "jr.json"),
         "--activation-path", data, "--layer", "1", "--top-k", "3", "--max-batches", "2", "--batch-size-tokens", "64",
         "--output-dir", str(root / "top"), "--device", "cpu")
    assert os.listdir(root / "top")


def test_scramble_compress_compare(workdir):
    root, data = workdir
    scr = _run("scramble_dataset.py", "--input-dir", data, "--output-dir", str(root / "scr"), "--chunk-tokens", "200", "--seed", "3").strip()
    from crosslayer_coding_b200.io import hdf5, manifest

    meta = json.load(open(os.path.join(scr, "metadata.json")))
    assert meta["scramble_seed"] == 3 and manifest.read_index(os.path.join(scr, "index.bin"), 512) == {0: 200, 1: 200, 2: 112}
    def all_rows(d, n):
        rows = []
        for c in range(n):
            with hdf5.open_chunk(d, c) as f:
                rows.append(np.concatenate([f["layer_0/inputs"].read_all(), f["layer_1/targets"].read_all()], axis=1))
        return np.concatenate(rows)
    a, b = all_rows(data, 4), all_rows(scr, 3)
    assert a.shape == b.shape and not np.array_equal(a, b)
    assert np.array_equal(a[np.lexsort(a.T[::-1])], b[np.lexsort(b.T[::-1])])  # same rows, layers kept aligned
    comp = _run("compress_activation_dataset.py", "--input-dir", data, "--output-dir", str(root / "gz")).strip()
    assert np.array_equal(all_rows(comp, 4), a)
    out = _run("compare_norm_stats.py", os.path.join(data, "norm_stats.json"), os.path.join(scr, "norm_stats.json"), "--tolerance", "1e-9")
    assert "max_abs_diff" in out


def test_two_rank_smoke_run_on_gloo(tmp_path):
    """scripts/smoke_train.py under torch.distributed.run with two Gloo ranks: the whole tensor-parallel training loop
    (sharded model, evaluation, distributed checkpoint with merge, final save) on the autograd step."""
    import json
    import subprocess
    import sys

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CLT_SMOKE_DIR=str(tmp_path), CLT_SMOKE_STEPS="8", CLT_SMOKE_TOKENS="16384", MASTER_ADDR="127.0.0.1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29537", os.path.join(repo, "scripts", "smoke_train.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    run = os.path.join(str(tmp_path), "run")
    names = set(os.listdir(run))
    assert {"metrics.json", "cfg.json", "latest", "final"} <= names, sorted(names)
    assert {"model.safetensors", "rank_0_model.safetensors", "rank_1_model.safetensors", "shard_meta.json"} <= set(os.listdir(os.path.join(run, "latest")))
    metrics = json.load(open(os.path.join(run, "metrics.json")))
    assert metrics["eval_metrics"] and all(v["total"] == v["total"] for v in metrics["train_losses"])
