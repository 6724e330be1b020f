"""The whole training loop on the fused engine (GPU): stores on disk, evaluation, asynchronous checkpoints, resume.

The CPU suite covers the same loop on the autograd step; here the optimizer state lives in the engine (moments, step
counter, dead-feature counters, step control block) and checkpoints are snapshotted on a side stream and written by a
thread while training goes on.
"""
import json
import os

import pytest

from crosslayer_coding_b200 import CLTConfig, TrainingConfig
from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset
from crosslayer_coding_b200.training.trainer import CLTTrainer

pytestmark = pytest.mark.gpu

L, D, F, B = 3, 64, 256, 128


def _dataset(tmp_path, tokens=2048):
    spec = SyntheticSpec(num_layers=L, d_model=D, dict_size=4 * D, active_mean=5, seed=0)
    return write_synthetic_dataset(str(tmp_path / "ds"), spec, total_tokens=tokens, chunk_tokens=512, dtype="bfloat16", device="cuda:0")


def _configs(path, steps, ckpt, **kw):
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=D, activation_fn="batchtopk", batchtopk_k=8, clt_dtype="bfloat16",
                    decoder_tying=kw.pop("tying", "none"))
    tc = TrainingConfig(learning_rate=2e-3, training_steps=steps, train_batch_size_tokens=B, activation_path=path, activation_dtype="bfloat16",
                        precision="bf16", normalization_method="mean_std", eval_interval=8, checkpoint_interval=ckpt, log_interval=4,
                        engine="fused", aux_loss_factor=1 / 32, dead_feature_window=10, async_checkpoint=True, **kw)
    return cfg, tc


def test_fused_training_run_writes_the_run_directory(tmp_path):
    cfg, tc = _configs(_dataset(tmp_path), steps=24, ckpt=8)
    log_dir = str(tmp_path / "run")
    tr = CLTTrainer(cfg, tc, log_dir=log_dir, device="cuda:0")
    assert tr.engine is not None
    tr.train()
    tr.engine.check_status()
    names = set(os.listdir(log_dir))
    for want in ("cfg.json", "metrics.json", "clt_checkpoint_8.safetensors", "clt_checkpoint_16.safetensors",
                 "clt_checkpoint_latest.safetensors", "trainer_state_latest.pt", "final"):
        assert want in names, (want, sorted(names))
    metrics = json.load(open(os.path.join(log_dir, "metrics.json")))
    losses = [v["total"] for v in metrics["train_losses"]]
    assert len(losses) >= 6 and all(x == x for x in losses)
    # the total takes the auxiliary term in once features count as dead (window of 10 steps): judge the reconstruction
    recon = [v["reconstruction"] for v in metrics["train_losses"]]
    assert recon[-1] < recon[0], (recon, losses)
    ev = metrics["eval_metrics"][-1]
    for key in ("reconstruction/explained_variance", "reconstruction/normalized_mean_reconstruction_error", "sparsity/avg_l0", "dead_features/total_eval"):
        assert key in ev, sorted(ev)
    # with a dead-feature window of 10 steps some of the 768 features have died and the auxiliary term ran
    assert any(v.get("auxiliary", 0.0) > 0.0 for v in metrics["train_losses"]) or ev["dead_features/total_eval"] == 0


@pytest.mark.parametrize("tying", ["none", "per_source"])
def test_fused_resume_equals_continuous(tmp_path, tying):
    path = _dataset(tmp_path)
    cfg, tc = _configs(path, steps=16, ckpt=1000, tying=tying)
    cont = CLTTrainer(cfg, tc, log_dir=str(tmp_path / "cont"), device="cuda:0")
    cont.train()
    cfg1, tc1 = _configs(path, steps=16, ckpt=8, tying=tying)
    first = CLTTrainer(cfg1, tc1, log_dir=str(tmp_path / "first"), device="cuda:0")
    orig_save = first.save_checkpoint

    def save_then_stop(step, final=False):
        orig_save(step, final)
        if step == 8 and not final:
            raise KeyboardInterrupt

    first.save_checkpoint = save_then_stop
    first.train()
    cfg2, tc2 = _configs(path, steps=16, ckpt=1000, tying=tying)
    resumed = CLTTrainer(cfg2, tc2, log_dir=str(tmp_path / "res"), device="cuda:0",
                         resume_from_checkpoint_path=os.path.join(str(tmp_path / "first"), "clt_checkpoint_8.safetensors"))
    assert resumed.start_step == 9
    assert resumed.engine.opt_step == first.engine.opt_step == 9
    resumed.train()
    for (n, a), (_, b) in zip(cont.model.named_parameters(), resumed.model.named_parameters()):
        # the same kernels on the same data; sums formed with atomics may differ in their last bits
        diff = (a.float() - b.float()).abs()
        assert float((diff > 0.02 * a.float().abs() + 2e-3).float().mean()) < 1e-3, (n, float(diff.max()))
