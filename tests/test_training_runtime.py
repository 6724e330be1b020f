import json
import os

import pytest
import torch

from crosslayer_coding_b200.models.base import shard_width
from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
from crosslayer_coding_b200.activation_generation.synthetic import SparseDictionarySynth, SyntheticSpec, write_synthetic_dataset
from crosslayer_coding_b200.training.checkpointing import CheckpointManager, merge_shards, slice_for_rank
from crosslayer_coding_b200.training.data import InMemoryActivationStore
from crosslayer_coding_b200.training.evaluator import CLTEvaluator
from crosslayer_coding_b200.training.trainer import CLTTrainer, learning_rate_at

L, D, F, B = 2, 8, 32, 16


def _dataset(tmp_path, tokens=256):
    spec = SyntheticSpec(num_layers=L, d_model=D, dict_size=24, active_mean=3, seed=0)
    return write_synthetic_dataset(str(tmp_path / "ds"), spec, total_tokens=tokens, chunk_tokens=64, dtype="float32")


def _configs(path, steps=10, **kw):
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=D, activation_fn=kw.pop("activation_fn", "relu"), **kw.pop("clt", {}))
    tc = TrainingConfig(learning_rate=1e-2, training_steps=steps, train_batch_size_tokens=B, activation_path=path,
                        activation_dtype="float32", normalization_method="mean_std", eval_interval=5, checkpoint_interval=kw.pop("ckpt", 100),
                        log_interval=2, **kw)
    return cfg, tc


def test_lr_schedules():
    mk = lambda **kw: TrainingConfig(learning_rate=1.0, training_steps=100, activation_path="x", **kw)  # noqa: E731
    assert learning_rate_at(mk(lr_scheduler="linear"), 0) == 1.0
    assert abs(learning_rate_at(mk(lr_scheduler="linear"), 100) - 0.1) < 1e-12
    assert abs(learning_rate_at(mk(lr_scheduler="cosine"), 50) - 0.5) < 1e-12
    f20 = mk(lr_scheduler="linear_final20")
    assert learning_rate_at(f20, 79) == 1.0 and abs(learning_rate_at(f20, 90) - 0.5) < 1e-12
    assert learning_rate_at(mk(lr_scheduler=None), 77) == 1.0


def test_training_run_writes_the_run_directory(tmp_path):
    cfg, tc = _configs(_dataset(tmp_path), steps=8, ckpt=4)
    log_dir = str(tmp_path / "run")
    tr = CLTTrainer(cfg, tc, log_dir=log_dir, device="cpu")
    tr.train()
    names = set(os.listdir(log_dir))
    for want in ("cfg.json", "metrics.json", "clt_checkpoint_4.safetensors", "clt_checkpoint_7.safetensors",
                 "clt_checkpoint_latest.safetensors", "trainer_state_latest.pt", "activation_store_latest.pt", "final"):
        assert want in names, (want, names)
    metrics = json.load(open(os.path.join(log_dir, "metrics.json")))
    assert len(metrics["train_losses"]) == 8 and metrics["eval_metrics"]
    ev = metrics["eval_metrics"][-1]
    for key in ("reconstruction/explained_variance", "reconstruction/normalized_mean_reconstruction_error", "sparsity/avg_l0",
                "layerwise/normalized_mse", "dead_features/total_eval", "layerwise/preactivation_std_dev"):
        assert key in ev
    assert all(v["total"] == v["total"] for v in metrics["train_losses"])  # finite, logged every step
    saved_cfg = json.load(open(os.path.join(log_dir, "cfg.json")))
    assert saved_cfg["normalization_method"] == "mean_std" and saved_cfg["num_features"] == F


@pytest.mark.parametrize("activation_fn,clt", [("relu", {}), ("batchtopk", {"batchtopk_k": 4})])
def test_resume_equals_continuous(tmp_path, activation_fn, clt):
    path = _dataset(tmp_path)
    cfg, tc = _configs(path, steps=10, ckpt=100, activation_fn=activation_fn, clt=clt)
    cont = CLTTrainer(cfg, tc, log_dir=str(tmp_path / "cont"), device="cpu")
    cont.train()
    cfg1, tc1 = _configs(path, steps=10, ckpt=6, activation_fn=activation_fn, clt=clt)
    first = CLTTrainer(cfg1, tc1, log_dir=str(tmp_path / "first"), device="cpu")
    # stop after step 6 by training with the loop bounded through a copy of the config
    first.training_config.training_steps = 10
    orig_save = first.save_checkpoint

    class Stop(Exception):
        pass

    def save_then_stop(step, final=False):
        orig_save(step, final)
        if step == 6 and not final:
            raise KeyboardInterrupt

    first.save_checkpoint = save_then_stop
    first.train()
    cfg2, tc2 = _configs(path, steps=10, ckpt=100, activation_fn=activation_fn, clt=clt)
    resumed = CLTTrainer(cfg2, tc2, log_dir=str(tmp_path / "res"), device="cpu",
                         resume_from_checkpoint_path=os.path.join(str(tmp_path / "first"), "clt_checkpoint_6.safetensors"))
    assert resumed.start_step == 7
    resumed.train()
    for (n, a), (_, b) in zip(cont.model.named_parameters(), resumed.model.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6), n


def test_checkpoint_io_error_is_logged_not_raised(tmp_path, monkeypatch):
    cfg, tc = _configs("x")
    m = CrossLayerTranscoder(cfg)
    cm = CheckpointManager(m, None, None, str(tmp_path), False, 0, torch.device("cpu"))
    import crosslayer_coding_b200.training.checkpointing as ck

    def boom(*a, **k):
        raise OSError("disk full")

    monkeypatch.setattr(ck, "save_safetensors_file", boom)
    cm._save_checkpoint(3, {"step": 3})  # must not raise


def test_distributed_checkpoint_layout_merge_and_reshard(tmp_path, monkeypatch):
    """Two simulated ranks save into one directory; the merged model equals the full model and a
    different world size can load it (ranks are simulated in-process, barriers patched out)."""
    cfg = CLTConfig(num_features=30, num_layers=2, d_model=4, activation_fn="jumprelu", decoder_tying="per_source",
                    enable_feature_offset=True, enable_feature_scale=True)
    full = CrossLayerTranscoder(cfg)
    with torch.no_grad():
        for p in full.parameters():
            p.normal_()
    full_sd = {k: v.clone() for k, v in full.state_dict().items()}
    import crosslayer_coding_b200.training.checkpointing as ck

    monkeypatch.setattr(ck.CheckpointManager, "_barrier", lambda self: None)

    class FakeModel(CrossLayerTranscoder):
        def __init__(self, cfg, rank, world):
            self._fake = (rank, world)
            super().__init__(cfg)

    def sharded(rank, world):
        m = CrossLayerTranscoder(cfg)
        m.world_size, m.rank = world, rank
        m.local_features = shard_width(30, world)
        m.feature_start = rank * m.local_features
        m.valid_features = max(0, min(30, m.feature_start + m.local_features) - m.feature_start)
        sd = slice_for_rank(full_sd, rank, world, 30)
        # rebuild parameters at shard width
        Fl = m.local_features
        m.enc_weight = torch.nn.Parameter(torch.zeros(2, Fl, 4))
        m.enc_bias = torch.nn.Parameter(torch.zeros(2, Fl))
        m.dec_weight = torch.nn.ParameterList([torch.nn.Parameter(torch.zeros(Fl, 1, 4)) for _ in range(2)])
        m.feature_offset = torch.nn.Parameter(torch.zeros(2, Fl))
        m.feature_scale = torch.nn.Parameter(torch.zeros(2, Fl))
        m.log_threshold = torch.nn.Parameter(torch.zeros(2, Fl))
        m.load_state_dict(sd)
        return m

    models = [sharded(r, 2) for r in range(2)]
    for r in (1, 0):  # rank 0 merges, so it goes last
        cm = CheckpointManager(models[r], None, None, str(tmp_path), True, r, torch.device("cpu"), world_size=2)
        cm._save_checkpoint(5, {"step": 5}, {"enc_m": torch.full((2, 16, 4), float(r)), "dec_m.0": torch.full((16, 1, 4), float(r)),
                                             "dead_counter": torch.arange(32) + 100 * r, "decb_m": torch.ones(2, 4), "step": torch.tensor(7)})
    step_dir = tmp_path / "step_5"
    names = set(os.listdir(step_dir))
    assert {"rank_0_model.safetensors", "rank_1_model.safetensors", "rank_0_optim.safetensors", "rank_1_optim.safetensors",
            "model.safetensors", "trainer_state.pt", "shard_meta.json"} <= names
    assert (tmp_path / "latest" / "model.safetensors").exists()
    from safetensors.torch import load_file

    merged = load_file(str(step_dir / "model.safetensors"))
    for k, v in full_sd.items():
        assert torch.equal(merged[k], v), k  # log_threshold / affine merged along the feature axis, padding dropped
    # same world size: own shard + own optimizer shard
    back = sharded(1, 2)
    with torch.no_grad():
        back.enc_weight.zero_()
    state = CheckpointManager(back, None, None, str(tmp_path), True, 1, torch.device("cpu"), world_size=2).load_checkpoint(str(step_dir))
    assert torch.equal(back.enc_weight, models[1].enc_weight) and float(state["optimizer_tensors"]["enc_m"].mean()) == 1.0
    # different world size: re-sharded from the merged file
    three = sharded(2, 3)
    with torch.no_grad():
        three.enc_weight.zero_()
    CheckpointManager(three, None, None, str(tmp_path), True, 2, torch.device("cpu"), world_size=3).load_checkpoint(str(step_dir))
    state3 = CheckpointManager(three, None, None, str(tmp_path), True, 2, torch.device("cpu"), world_size=3).load_checkpoint(str(step_dir))
    want = slice_for_rank(full_sd, 2, 3, 30)
    assert torch.equal(three.state_dict()["encoder_module.encoders.1.weight"], want["encoder_module.encoders.1.weight"])
    # ... and so are the optimizer tensors: rank 2 of 3 holds features [32, 30) -> nothing valid; rank 1 of 3 holds [16, 30)
    ot = CheckpointManager(sharded(1, 3), None, None, str(tmp_path), True, 1, torch.device("cpu"), world_size=3).load_checkpoint(str(step_dir))["optimizer_tensors"]
    assert ot["enc_m"].shape == (2, 16, 4) and float(ot["enc_m"][:, :14].mean()) == 1.0 and float(ot["enc_m"][:, 14:].abs().sum()) == 0.0
    assert ot["dec_m.0"].shape == (16, 1, 4) and float(ot["dec_m.0"][:14].mean()) == 1.0
    # saved rank 1 counted 100 + l * 16 + j for its local feature j of layer l: global feature 16 + j
    assert ot["dead_counter"].shape == (32,) and int(ot["dead_counter"][0]) == 100 and int(ot["dead_counter"][16 + 3]) == 100 + 16 + 3
    assert int(ot["step"]) == 7 and torch.equal(ot["decb_m"], torch.ones(2, 4))
    assert state3["optimizer_resharded_from"] == 2
    # one world: everything concatenated, padding dropped
    one = CheckpointManager(sharded(0, 1), None, None, str(tmp_path), False, 0, torch.device("cpu"), world_size=1).load_checkpoint(str(step_dir))["optimizer_tensors"]
    assert one["enc_m"].shape == (2, 30, 4) and float(one["enc_m"][:, :16].sum()) == 0.0 and float(one["enc_m"][:, 16:].mean()) == 1.0
    # pruning keeps the newest three step directories
    cm0 = CheckpointManager(models[0], None, None, str(tmp_path), True, 0, torch.device("cpu"), world_size=1)
    for s in (6, 7, 8):
        os.makedirs(tmp_path / f"step_{s}", exist_ok=True)
    cm0._prune_old()
    assert sorted(d for d in os.listdir(tmp_path) if d.startswith("step_")) == ["step_6", "step_7", "step_8"]


def test_evaluator_metric_definitions():
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=D, activation_fn="relu")
    m = CrossLayerTranscoder(cfg)
    ev = CLTEvaluator(m, torch.device("cpu"))
    x = {l: torch.randn(20, D) for l in range(L)}
    y = {l: torch.randn(20, D) for l in range(L)}
    dead = torch.zeros(L, F, dtype=torch.bool)
    dead[0, :5] = True
    out = ev.compute_metrics(x, y, dead)
    recon = m(x)
    acts = m.get_feature_activations(x)
    nmse0 = ((recon[0] - y[0]) ** 2).mean() / y[0].var(dim=0, unbiased=False).mean()
    assert abs(out["layerwise/normalized_mse"]["layer_0"] - float(nmse0)) < 1e-5
    l0 = float((acts[1] != 0).float().sum(dim=1).mean())
    assert abs(out["layerwise/l0"]["layer_1"] - l0) < 1e-5
    assert abs(out["sparsity/avg_l0"] - out["sparsity/total_l0"] / L) < 1e-6
    assert out["layerwise/dead_features"]["layer_0"] == 5 and out["dead_features/total_eval"] == 5
    assert len(out["layerwise/log_feature_density"]["layer_0"]) == F
    assert 0.0 <= out["reconstruction/explained_variance"] <= 1.0


def test_in_memory_store_and_fused_engine_gate():
    from crosslayer_coding_b200.training.fused_engine import engine_supports

    cfg = CLTConfig(num_features=F, num_layers=L, d_model=D, activation_fn="batchtopk", batchtopk_k=2, clt_dtype="bfloat16")
    tc = TrainingConfig(learning_rate=1e-3, training_steps=5, activation_path="x", preactivation_coef=0.0, precision="bf16")
    assert engine_supports(cfg, tc) is None
    assert engine_supports(CLTConfig(num_features=F, num_layers=L, d_model=D + 1, activation_fn="relu"), tc) is not None  # d_model % 8
    # gradient clipping, ReLU and fp16 (with fp16 weights) are covered by the fused step
    assert engine_supports(cfg, TrainingConfig(learning_rate=1e-3, training_steps=5, activation_path="x",
                                               preactivation_coef=0.0, gradient_clip_val=1.0)) is None
    assert engine_supports(CLTConfig(num_features=F, num_layers=L, d_model=D, activation_fn="relu", clt_dtype="bfloat16"), tc) is None
    assert engine_supports(CLTConfig(num_features=F, num_layers=L, d_model=D, activation_fn="batchtopk", batchtopk_k=2, topk_mode="per_layer"), tc) is not None
    pool = torch.randn(3, 2, L, B, D)
    st = InMemoryActivationStore(pool, "cpu", loop=False)
    got = [x.stacked.clone() for x, _ in st]
    assert len(got) == 3 and torch.equal(got[2], pool[2, 0])
