"""CPU checks of the benchmark's contract and of the rules that decide which step implementation a configuration gets."""
import json
import os
import subprocess
import sys

import pytest
import torch

from crosslayer_coding_b200 import CLTConfig, TrainingConfig
from crosslayer_coding_b200.training.checkpointing import optimizer_shard_axis, reshard_optimizer_tensors
from crosslayer_coding_b200.training.fused_engine import engine_supports

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tc(**kw):
    base = dict(learning_rate=1e-3, training_steps=10, activation_path="unused", aux_loss_factor=0.0)
    base.update(kw)
    return TrainingConfig(**base)


def test_fused_step_covers_the_reference_configurations():
    ok = dict(num_features=64, num_layers=2, d_model=16, batchtopk_k=4, topk_k=4)
    for fn in ("batchtopk", "topk", "jumprelu", "relu"):
        for tying in ("none", "per_source", "per_target"):
            assert engine_supports(CLTConfig(activation_fn=fn, decoder_tying=tying, **ok), _tc()) is None, (fn, tying)
    assert engine_supports(CLTConfig(activation_fn="batchtopk", skip_connection=True, **ok), _tc(gradient_clip_val=1.0, preactivation_coef=0.1)) is None
    assert engine_supports(CLTConfig(activation_fn="batchtopk", **ok), _tc(precision="fp16")) is None
    # feature offset / scale of tied decoders: on the fused step unless JumpReLU or the auxiliary loss is in play
    aff = dict(decoder_tying="per_source", enable_feature_offset=True, enable_feature_scale=True, **ok)
    assert engine_supports(CLTConfig(activation_fn="batchtopk", **aff), _tc()) is None
    assert engine_supports(CLTConfig(activation_fn="relu", **aff), _tc()) is None
    assert "auxiliary" in engine_supports(CLTConfig(activation_fn="batchtopk", **aff), _tc(aux_loss_factor=1 / 32))
    assert "jumprelu" in engine_supports(CLTConfig(activation_fn="jumprelu", **aff), _tc())
    # what stays on the autograd step
    assert "per_layer" in engine_supports(CLTConfig(activation_fn="batchtopk", topk_mode="per_layer", **ok), _tc())
    assert "d_model" in engine_supports(CLTConfig(activation_fn="batchtopk", batchtopk_k=4, num_features=64, num_layers=2, d_model=20), _tc())
    assert "d_model" in engine_supports(CLTConfig(activation_fn="batchtopk", batchtopk_k=4, num_features=64, num_layers=2, d_model=4096), _tc())


def test_affine_moments_are_resharded_with_the_features():
    L, F = 2, 20
    per_rank = []
    for r in range(2):  # two ranks, shards of 16 columns (10 valid + padding on the second)
        per_rank.append({"foff_m": torch.arange(L * 16, dtype=torch.float32).view(L, 16) + 100 * r,
                         "fsc_v": torch.ones(L, 16) * (r + 1), "step": torch.tensor(7)})
    assert optimizer_shard_axis("foff_m", per_rank[0]["foff_m"]) == 1 and optimizer_shard_axis("step", per_rank[0]["step"]) is None
    out = reshard_optimizer_tensors(per_rank, F, L, 0, 1)
    assert out["foff_m"].shape[0] == L and out["foff_m"].shape[1] >= F
    assert torch.equal(out["foff_m"][:, :16], per_rank[0]["foff_m"]) and torch.equal(out["foff_m"][:, 16:20], per_rank[1]["foff_m"][:, :4])
    assert torch.equal(out["fsc_v"][:, 16:20], torch.full((L, 4), 2.0)) and int(out["step"]) == 7


def test_benchmark_arms_print_the_same_config_keys():
    sys.path.insert(0, REPO)
    import bench

    argv = sys.argv
    try:
        sys.argv = ["bench.py", "--decoder-tying", "per_source", "--precision", "fp16", "--dead-frac", "0.05"]
        args = bench.parse_args()
    finally:
        sys.argv = argv
    bench.MODEL.clear()
    bench.MODEL.update(bench.SHAPES["pythia-70m"])
    bench.MODEL["tying"] = "per_source"
    ours = bench.config_block(args, 8, False)
    args.impl = "reference"
    ref = bench.config_block(args, 8, False)
    assert ours == ref and ours["parallelism"] == "tp8" and "fp16" in ours["optimizer"] and "5%" in ours["loss"]
    assert bench.metric_name(False).startswith("train tokens/sec")


@pytest.mark.parametrize("impl", ["ours", "reference"])
def test_benchmark_reports_unavailable_without_a_gpu(impl):
    if torch.cuda.is_available():
        pytest.skip("CPU-only check")
    res = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", impl, "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == impl and "unavailable" in line
