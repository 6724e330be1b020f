"""Fused training step against the unmodified reference implementation over many steps (GPU).

Both arms start from the same weights and see the same batches of the seeded synthetic stream: the reference's own
``CrossLayerTranscoder`` + ``LossManager`` + ``torch.optim.AdamW`` (fp32 parameters, the step sequence of
clt/training/trainer.py:661-810) and this package's fused engine (bf16 weights, fp32 moments).  After 60 steps the
held-out normalised MSE of the two must agree within a few percent and both must have learned something.
The reference is the offline install under ``baseline/_ref``; the test is skipped where it is absent.
"""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_ROOT = os.path.join(REPO, "baseline", "_ref")


def _reference_modules():
    if not os.path.isdir(os.path.join(REF_ROOT, "clt")):
        pytest.skip("reference implementation is not installed under baseline/_ref")
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    try:
        from clt.config import CLTConfig as RefCLTConfig, TrainingConfig as RefTrainingConfig
        from clt.models.clt import CrossLayerTranscoder as RefCLT
        from clt.training.losses import LossManager as RefLossManager
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"reference import failed: {type(exc).__name__}: {exc}")
    return RefCLTConfig, RefTrainingConfig, RefCLT, RefLossManager


def _nmse(yhat, y):
    y = y.float()
    return float(((yhat.float() - y) ** 2).sum() / ((y - y.mean(dim=1, keepdim=True)) ** 2).sum())


@pytest.mark.parametrize("tying", ["none", "per_source"])
def test_fused_step_tracks_the_reference_over_60_steps(tying):
    RefCLTConfig, RefTrainingConfig, RefCLT, RefLossManager = _reference_modules()
    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from crosslayer_coding_b200.activation_generation.synthetic import SparseDictionarySynth, SyntheticSpec
    from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine

    dev = torch.device("cuda:0")
    L, d, F, B, k, steps, lr = 3, 64, 768, 512, 12, 60, 2e-3
    synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=4 * d, active_mean=6, seed=77), device=dev)
    synth.fit_norm_stats(4096)
    batches = [synth.sample(B, seed=500 + i, normalize=True, dtype=torch.bfloat16) for i in range(8)]
    held = synth.sample(1024, seed=9999, normalize=True, dtype=torch.bfloat16)
    common = dict(num_features=F, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=k, decoder_tying=tying)
    torch.manual_seed(3)
    ref = RefCLT(RefCLTConfig(**common), process_group=None, device=dev)
    if tying != "none":
        with torch.no_grad():  # tied decoders start at zero in the reference; give both arms the same non-zero start
            for name, p in ref.named_parameters():
                if "decoder_module.decoders" in name and name.endswith("weight"):
                    p.uniform_(-0.05, 0.05)
    ours = CrossLayerTranscoder(CLTConfig(clt_dtype="bfloat16", **common), device=dev)
    ours.load_state_dict({n: v.detach().clone() for n, v in ref.state_dict().items()})
    tkw = dict(learning_rate=lr, training_steps=steps, train_batch_size_tokens=B, activation_path="unused", normalization_method="none",
               sparsity_lambda=0.0, preactivation_coef=0.0, aux_loss_factor=0.0, optimizer="adamw", lr_scheduler=None)
    ref_tc = RefTrainingConfig(precision="fp32", **tkw)
    tc = TrainingConfig(precision="bf16", **tkw)
    loss_mgr = RefLossManager(ref_tc, clt_config=ref.config)
    opt = torch.optim.AdamW(ref.parameters(), lr=lr)
    eng = FusedBatchTopKEngine(ours, tc, B)
    ref_losses, our_losses = [], []
    for step in range(steps):
        x, y = batches[step % len(batches)]
        xin = {l: x[l].float() for l in range(L)}
        yin = {l: y[l].float() for l in range(L)}
        opt.zero_grad(set_to_none=True)
        acts = ref.get_feature_activations(xin)
        loss, parts = loss_mgr.compute_total_loss(ref, xin, yin, step, steps, precomputed_activations=acts)
        loss.backward()
        opt.step()
        if hasattr(ref, "decoder_module") and hasattr(ref.decoder_module, "_cached_decoder_norms"):
            ref.decoder_module._cached_decoder_norms = None
        ref_losses.append(float(parts["reconstruction"]))
        out = eng.train_step(x, y, step, lr)
        our_losses.append(float(out.reconstruction))
    eng.check_status()
    with torch.no_grad():
        ref_out = ref({l: held[0][l].float() for l in range(L)})
        ref_nmse = _nmse(torch.stack([ref_out[l] for l in range(L)]), held[1])
        our_nmse = _nmse(eng.forward(held[0][:, :B].contiguous(), held[1][:, :B].contiguous()), held[1][:, :B])
        ref_nmse_b = _nmse(torch.stack([ref_out[l][:B] for l in range(L)]), held[1][:, :B])
    assert ref_losses[-1] < 0.8 * ref_losses[0] and our_losses[-1] < 0.8 * our_losses[0], (ref_losses[::10], our_losses[::10])
    # the loss curves stay together step by step
    for a, b in zip(our_losses[::5], ref_losses[::5]):
        assert abs(a - b) < 0.03 * b + 1e-3, (our_losses[::5], ref_losses[::5])
    assert abs(our_nmse - ref_nmse_b) < 0.03 * ref_nmse_b + 1e-3, (our_nmse, ref_nmse_b, ref_nmse)
