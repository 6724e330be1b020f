import json
import math

import pytest
import torch

from crosslayer_coding_b200 import CLTConfig, TrainingConfig
from crosslayer_coding_b200.models import activations as act
from crosslayer_coding_b200.models.activations import BatchTopK, JumpReLU, TokenTopK


def test_clt_config_validation_and_json_roundtrip(tmp_path):
    with pytest.raises(ValueError):
        CLTConfig(num_features=8, num_layers=2, d_model=4, activation_fn="batchtopk")
    with pytest.raises(ValueError):
        CLTConfig(num_features=8, num_layers=2, d_model=4, activation_fn="topk")
    with pytest.raises(AssertionError):
        CLTConfig(num_features=0, num_layers=2, d_model=4)
    cfg = CLTConfig(num_features=8, num_layers=2, d_model=4, activation_fn="batchtopk", batchtopk_k=3, decoder_tying="per_source")
    p = tmp_path / "cfg.json"
    cfg.to_json(str(p))
    assert CLTConfig.from_json(str(p)) == cfg


def test_legacy_config_keys(tmp_path):
    raw = {"num_features": 8, "num_layers": 2, "d_model": 4, "normalization_method": "auto", "sqrt_d_model_normalize": False}
    p = tmp_path / "old.json"
    p.write_text(json.dumps(raw))
    cfg = CLTConfig.from_json(str(p))
    assert cfg.normalization_method == "mean_std" and cfg.decoder_tying == "none"
    raw["sqrt_d_model_normalize"] = True
    p.write_text(json.dumps(raw))
    assert CLTConfig.from_json(str(p)).normalization_method == "sqrt_d_model"


def test_training_config_accepts_auto_and_validates():
    tc = TrainingConfig(learning_rate=1e-3, training_steps=10, activation_path="x", normalization_method="auto")
    assert tc.normalization_method == "mean_std"
    with pytest.raises(AssertionError):
        TrainingConfig(learning_rate=1e-3, training_steps=10)  # local_manifest needs a path
    with pytest.raises(AssertionError):
        TrainingConfig(learning_rate=1e-3, training_steps=10, activation_source="remote", remote_config={"server_url": "u"})
    with pytest.raises(AssertionError):
        TrainingConfig(learning_rate=-1, training_steps=10, activation_path="x")


def test_batchtopk_mask_counts_and_values():
    x = torch.tensor([[1.0, 5.0, 2.0, 0.5], [4.0, 3.0, -1.0, 6.0]])
    m = BatchTopK._compute_mask(x, 1)
    assert int(m.sum()) == 2 and m[0, 1] and m[1, 3]
    assert int(BatchTopK._compute_mask(x, 0).sum()) == 0
    assert int(BatchTopK._compute_mask(x, 10).sum()) == x.numel()
    out = BatchTopK.apply(x, 2, True, None)
    assert torch.equal(out != 0, BatchTopK._compute_mask(x, 2))
    assert BatchTopK._compute_mask(torch.zeros(0, 4), 2).shape == (0, 4)


def test_batchtopk_separate_ranking_and_ste_backward():
    x = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], requires_grad=True)
    rank = -x.detach()
    out = BatchTopK.apply(x, 1, True, rank)
    assert torch.equal(out.detach(), torch.tensor([[1.0, 2.0, 0.0], [0.0, 0.0, 0.0]]))
    out.sum().backward()
    assert torch.equal(x.grad, torch.tensor([[1.0, 1.0, 0.0], [0.0, 0.0, 0.0]]))


def test_batchtopk_ties_prefer_lowest_flat_index():
    x = torch.ones(2, 4)
    m = BatchTopK._compute_mask(x, 1)  # keep 2 of 8 identical values
    assert torch.equal(m.flatten().nonzero().flatten(), torch.tensor([0, 1]))


def test_tokentopk_int_and_fraction():
    x = torch.tensor([[1.0, 5.0, 2.0, 0.5], [4.0, 3.0, -1.0, 6.0]])
    m = TokenTopK._compute_mask(x, 2)
    assert torch.equal(m, torch.tensor([[False, True, True, False], [True, False, False, True]]))
    m = TokenTopK._compute_mask(x, 0.5)
    assert torch.equal(m.sum(dim=1), torch.tensor([2, 2]))
    assert int(TokenTopK._compute_mask(x, 0).sum()) == 0
    assert int(TokenTopK._compute_mask(x, 100).sum()) == 8
    assert act.resolve_token_k(0.26, 8) == 3  # ceil(2.08)


@pytest.mark.parametrize("bw", [0.5, 1.0, 2.0])
def test_jumprelu_forward_backward_closed_form(bw):
    x = torch.tensor([[0.1, 0.5, 1.2], [0.9, 1.0, 2.0]], requires_grad=True)
    theta = torch.tensor([0.5, 1.0, 1.5], requires_grad=True)
    out = JumpReLU.apply(x, theta, bw)
    gate = (x.detach() >= theta.detach()).float()
    assert torch.equal(out.detach(), gate * x.detach())
    g = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    out.backward(g)
    assert torch.allclose(x.grad, g * gate)
    window = ((x.detach() - theta.detach()).abs() <= bw / 2).float()
    assert torch.allclose(theta.grad, (g * (-x.detach() / bw) * window).sum(dim=0))


def test_jumprelu_needs_input_grad_combinations():
    x = torch.randn(4, 3)
    theta = torch.rand(3, requires_grad=True)
    JumpReLU.apply(x, theta, 1.0).sum().backward()
    assert theta.grad is not None
    x2 = torch.randn(4, 3, requires_grad=True)
    JumpReLU.apply(x2, torch.rand(3), 1.0).sum().backward()
    assert x2.grad is not None


def test_global_batchtopk_ranks_on_zscores_and_keeps_original_values():
    torch.manual_seed(0)
    pre = {0: torch.randn(16, 8) * 10 + 3, 1: torch.randn(16, 8) * 0.1}
    out = act.apply_global_batchtopk(pre, 2)
    total = sum(int((o != 0).sum()) for o in out.values())
    assert total == 2 * 16
    # both layers contribute although their raw scales differ by 100x
    assert all(int((o != 0).sum()) > 4 for o in out.values())
    for l in pre:
        kept = out[l] != 0
        assert torch.equal(out[l][kept], pre[l][kept])
    assert act.apply_global_batchtopk(pre, None)[0].equal(pre[0])


def test_global_tokentopk_per_row_count():
    torch.manual_seed(1)
    pre = {0: torch.randn(10, 6), 1: torch.randn(10, 6)}
    out = act.apply_global_tokentopk(pre, 3)
    per_row = sum((o != 0).sum(dim=1) for o in out.values())
    assert torch.equal(per_row, torch.full((10,), 3))


def test_small_helpers_and_the_example_config():
    import json
    import os

    import numpy as np
    import torch

    from crosslayer_coding_b200 import CLTConfig
    from crosslayer_coding_b200.utils import format_elapsed_time, numpy_uint16_to_torch_bfloat16, torch_bfloat16_to_numpy_uint16

    assert format_elapsed_time(59.9) == "00:59" and format_elapsed_time(3725) == "01:02:05" and format_elapsed_time(90000) == "25:00:00"
    x = torch.tensor([[1.0, -2.5, 3.140625], [0.0, 65280.0, -0.0078125]]).bfloat16()
    bits = torch_bfloat16_to_numpy_uint16(x)
    assert bits.dtype == np.uint16 and bits.shape == (2, 3)
    assert bits[0, 0] == 0x3F80 and bits[0, 1] == 0xC020  # 1.0 and -2.5 as bf16 bit patterns
    assert torch.equal(numpy_uint16_to_torch_bfloat16(bits), x)
    with pytest.raises(TypeError):
        torch_bfloat16_to_numpy_uint16(torch.zeros(2))
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CLTConfig(**json.load(open(os.path.join(repo, "example_clt_config_gpt2_local.json"))))
    assert cfg.num_layers == 12 and cfg.activation_fn == "batchtopk" and cfg.batchtopk_k == 200
