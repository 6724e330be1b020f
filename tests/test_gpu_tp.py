"""Tensor-parallel fused step on 2 (and 4) GPUs against the single-GPU result.

Ranks run as child processes (one per GPU) with NVLS disabled in NCCL; the kernels use plain peer loads and
stores.  The selection must be identical for every world size (global k*B entries, lowest-flat-index
tie-break), losses and updated weights must agree within bf16 tolerance.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world: int, out: str, features: int, port: int, lam: float = 0.0, activation: str = "batchtopk", extra=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    worker = os.path.join(HERE, "tp_worker.py")
    args = ["--out", out, "--features", str(features), "--lam", str(lam), "--activation", activation, *extra]
    if world == 1:
        cmd = [sys.executable, worker, *args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), worker, *args]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return torch.load(out, weights_only=False)


@pytest.mark.parametrize("world,features,lam", [(2, 512, 0.0), (2, 520, 0.0), (2, 512, 0.02), (4, 512, 0.0), (4, 520, 0.02), (8, 512, 0.02)])
def test_tp_matches_single_gpu(tmp_path, world, features, lam):
    """520 features over 2 or 4 ranks: shards are padded to a multiple of 8 columns (264 / 136), the last rank holds fewer
    valid features than the others."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ref = _run(1, str(tmp_path / "w1.pt"), features, 29611, lam)
    got = _run(world, str(tmp_path / f"w{world}.pt"), features, 29613 + world, lam)
    assert got["entries"] == ref["entries"], (got["entries"], ref["entries"])
    assert got["staging_ok"] and ref["staging_ok"], "sharded staging returned a different batch"
    assert got["h2d_bytes_per_rank"] * world == got["h2d_bytes"]
    for a, b in zip(got["losses"], ref["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (got["losses"], ref["losses"])
    for key, w_ref in ref["state"].items():
        w = got["state"][key]
        assert w.shape == w_ref.shape, key
        bad = ((w - w_ref).abs() > 0.01 * w_ref.abs() + 4e-4).float().mean().item()
        assert bad < 5e-3, (key, bad, (w - w_ref).abs().max().item())


def test_tp_jumprelu_matches_single_gpu(tmp_path):
    """Natively trained JumpReLU under tensor parallelism: thresholds, selection and the threshold-gradient GEMM are
    all local to the feature shard; only the decode partials and the gradient seed cross NVLink."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ref = _run(1, str(tmp_path / "w1.pt"), 512, 29631, 0.02, "jumprelu")
    got = _run(2, str(tmp_path / "w2.pt"), 512, 29633, 0.02, "jumprelu")
    assert got["entries"] == ref["entries"] and ref["entries"][0] > 0, (got["entries"], ref["entries"])
    for a, b in zip(got["losses"], ref["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (got["losses"], ref["losses"])
    for key, w_ref in ref["state"].items():
        w = got["state"][key]
        assert w.shape == w_ref.shape, key
        bad = ((w - w_ref).abs() > 0.01 * w_ref.abs() + 2e-3).float().mean().item()
        assert bad < 5e-3, (key, bad)


@pytest.mark.parametrize("extra,activation,lam", [
    (("--dtype", "float16"), "batchtopk", 0.02),                       # fp16 weights + loss scaling, found-inf flag agreed across ranks
    (("--tying", "per_source"), "jumprelu", 0.02),                      # tied JumpReLU: threshold-gradient GEMM on the summed seed
    (("--tying", "per_target", "--clip", "0.05"), "batchtopk", 0.02),   # global-norm clipping: norm summed across ranks in the control kernel
    (("--tying", "per_source", "--affine"), "batchtopk", 0.0),           # feature offset / scale: sharded with the features
    (("--dead",), "batchtopk", 0.0),                                      # auxiliary loss, dead features on one shard only / on all shards
    (("--dead", "--aux-unfused"), "batchtopk", 0.0),                     # the same through the per-layer PyTorch form of the term
])
def test_tp_variants_match_single_gpu(tmp_path, extra, activation, lam):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ref = _run(1, str(tmp_path / "w1.pt"), 512, 29651, lam, activation, extra)
    got = _run(2, str(tmp_path / "w2.pt"), 512, 29653, lam, activation, extra)
    assert got["entries"] == ref["entries"], (got["entries"], ref["entries"])
    assert got["skipped"] == ref["skipped"]
    for a, b in zip(got["losses"], ref["losses"]):
        assert abs(a - b) < 3e-3 * max(1.0, abs(b)), (got["losses"], ref["losses"])
    for a, b in zip(got["grad_norms"], ref["grad_norms"]):
        assert abs(a - b) < 2e-2 * max(1e-6, abs(b)), (got["grad_norms"], ref["grad_norms"])
    for key, w_ref in ref["state"].items():
        w = got["state"][key]
        assert w.shape == w_ref.shape, key
        bad = ((w - w_ref).abs() > 0.01 * w_ref.abs() + 2e-3).float().mean().item()
        assert bad < 5e-3, (key, bad)


@pytest.mark.parametrize("world,features", [(2, 512), (2, 520), (4, 512)])
def test_tp_token_topk_equals_single_gpu_selection(tmp_path, world, features):
    """Per-token top-k across feature shards: local top k, composite keys to the token owners, cut published to every
    rank.  The selection equals the single-GPU one entry for entry (k per token, ties by the lowest flat index)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ref = _run(1, str(tmp_path / "w1.pt"), features, 29671, 0.0, "topk")
    got = _run(world, str(tmp_path / f"w{world}.pt"), features, 29673 + world, 0.0, "topk")
    assert len(ref["selection"]) == 128 * 8
    assert got["selection"] == ref["selection"]
    assert got["entries"] == ref["entries"], (got["entries"], ref["entries"])
    for a, b in zip(got["losses"], ref["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (got["losses"], ref["losses"])
    for key, w_ref in ref["state"].items():
        w = got["state"][key]
        bad = ((w - w_ref).abs() > 0.01 * w_ref.abs() + 4e-4).float().mean().item()
        assert bad < 5e-3, (key, bad)


def test_tp_trainer_loop_with_owner_only_targets(tmp_path):
    """CLTTrainer.train() on 2 GPUs with the fused engine: sharded staging where the targets stay with the token owners,
    evaluation (which gathers the owners' rows again), asynchronous distributed checkpoints."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    if os.environ.get("CLT_RUN_UNVERIFIED", "") in ("", "0"):
        # Its only run so far used a worker that kept using the process group after the trainer had destroyed it and ran into
        # the time limit; the worker now owns the group, but the test has not completed once on a 2-GPU box since.
        pytest.skip("not yet completed once on a 2-GPU box (set CLT_RUN_UNVERIFIED=1 to run it)")
    import json

    from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset

    data = write_synthetic_dataset(str(tmp_path / "ds"), SyntheticSpec(num_layers=3, d_model=64, dict_size=256, active_mean=5, seed=0),
                                   total_tokens=2048, chunk_tokens=512, dtype="bfloat16", device="cuda:0")
    out = str(tmp_path / "out.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29691",
           os.path.join(HERE, "tp_trainer_worker.py"), "--data", data, "--log-dir", str(tmp_path / "run"), "--out", out]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    got = json.load(open(out))
    assert got["owner_only"], "the trainer did not restrict the staging of the targets"
    assert got["targets_ok"], "evaluation would not see the same targets as an unsharded store"
    assert got["recon"][-1] < got["recon"][0], got["recon"]
    ev = got["eval"]
    assert 0.0 < ev["reconstruction/normalized_mean_reconstruction_error"] < 1.5, ev
    for want in ("clt_checkpoint_8", "latest", "final", "metrics.json"):
        assert any(want in name for name in got["files"]), (want, got["files"])
