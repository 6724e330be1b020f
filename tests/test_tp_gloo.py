"""Tensor-parallel equivalence on CPU (Gloo, 2 and 3 ranks as spawned processes): a model built from the same
full weights gives the same forward, the same loss terms and, after gathering shards, the same gradients as
the single-process model, for every activation function.  BatchTopK keeps exactly k*B entries at every
world size."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
from crosslayer_coding_b200.training.checkpointing import merge_shards, slice_for_rank
from crosslayer_coding_b200.training.losses import LossManager

L, D, F, B = 3, 8, 22, 12  # F is not divisible by 3: the last rank carries padding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _config(fn, tying):
    kw = dict(num_features=F, num_layers=L, d_model=D, activation_fn=fn, decoder_tying=tying)
    if fn == "batchtopk":
        kw["batchtopk_k"] = 5
    if fn == "topk":
        kw["topk_k"] = 0.25
    if tying != "none":
        kw.update(enable_feature_offset=True, enable_feature_scale=True, skip_connection=True)
    return CLTConfig(**kw)


def _full_state(cfg):
    torch.manual_seed(0)
    m = CrossLayerTranscoder(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(torch.randn_like(p) * 0.3)
        if m.log_threshold is not None:
            m.log_threshold.fill_(-2.0)
    return {k: v.clone() for k, v in m.state_dict().items()}


def _data():
    g = torch.Generator().manual_seed(1)
    x = {l: torch.randn(B, D, generator=g) for l in range(L)}
    y = {l: torch.randn(B, D, generator=g) for l in range(L)}
    return x, y


def _tc():
    return TrainingConfig(learning_rate=1e-3, training_steps=10, activation_path="x", normalization_method="none",
                          sparsity_lambda=0.3, preactivation_coef=0.05, aux_loss_factor=0.5)


def _run_model(cfg, state, group, rank, world):
    model = CrossLayerTranscoder(cfg, process_group=group)
    model.load_state_dict(slice_for_rank(state, rank, world, F) if world > 1 else state)
    x, y = _data()
    lm = LossManager(_tc())
    dead = torch.zeros(L, F, dtype=torch.bool)
    dead[1, ::3] = True
    loss, parts, acts = lm.compute_total_loss_tensors(model, x, y, 5, 10, dead_neuron_mask=dead)
    loss.backward()
    recon = model(x)
    grads = {}
    sd_keys = model.state_dict(keep_vars=True)
    # map gradients to reference key names through a state_dict-shaped view of .grad
    gm = CrossLayerTranscoder(cfg, process_group=group)
    with torch.no_grad():
        for (n, p), (_, q) in zip(model.named_parameters(), gm.named_parameters()):
            q.copy_(p.grad if p.grad is not None else torch.zeros_like(p))
    grads = {k: v.clone() for k, v in gm.state_dict().items()}
    n_active = sum(int((a != 0).sum()) for a in acts.values())
    full_acts = model.get_feature_activations(x, gather=True)
    return {"parts": {k: float(v) for k, v in parts.items()}, "recon": {l: r.detach() for l, r in recon.items()},
            "grads": grads, "n_active": n_active, "acts": {l: a.detach() for l, a in full_acts.items()}}


def _worker(rank, world, port, fn, tying, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = _config(fn, tying)
        res = _run_model(cfg, _full_state(cfg), dist.group.WORLD, rank, world)
        n = torch.tensor([res["n_active"]])
        dist.all_reduce(n)
        gathered = [None] * world
        dist.all_gather_object(gathered, res["grads"])
        if rank == 0:
            res["grads"] = merge_shards(gathered, F)
            res["n_active"] = int(n)
            torch.save(res, out_path)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("fn,tying", [("relu", "none"), ("jumprelu", "none"), ("batchtopk", "none"), ("topk", "none"),
                                      ("batchtopk", "per_source"), ("jumprelu", "per_target")])
def test_tp_equivalence(world, fn, tying):
    if world == 3 and (fn, tying) not in (("batchtopk", "none"), ("jumprelu", "per_target")):
        pytest.skip("3-rank (padded shard) run only for two representative configurations")
    cfg = _config(fn, tying)
    ref = _run_model(cfg, _full_state(cfg), None, 0, 1)
    out = os.path.join(tempfile.mkdtemp(), "tp.pt")
    mp.spawn(_worker, args=(world, _free_port(), fn, tying, out), nprocs=world, join=True)
    got = torch.load(out, weights_only=False)
    if fn == "batchtopk":
        assert got["n_active"] == ref["n_active"] == 5 * B  # exactly k*B at every world size
    for l in range(L):
        assert torch.allclose(got["recon"][l], ref["recon"][l], atol=1e-5), l
        assert torch.equal(got["acts"][l] != 0, ref["acts"][l] != 0), l
    for k, v in ref["parts"].items():
        assert abs(got["parts"][k] - v) < 1e-4 * max(1.0, abs(v)), (k, got["parts"][k], v)
    for k, g in ref["grads"].items():
        assert torch.allclose(got["grads"][k], g, atol=2e-5), (k, (got["grads"][k] - g).abs().max())


def _ops_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from crosslayer_coding_b200.parallel import ops

        t = torch.full((3,), float(rank + 1))
        ops.all_reduce(t)
        assert torch.equal(t, torch.full((3,), 3.0))
        local = torch.arange(4.0).reshape(1, 4) + 10 * rank
        local.requires_grad_(True)
        full = ops.gather_cols(local, 7)
        assert full.shape == (1, 7) and float(full[0, 4]) == 10.0
        full.sum().backward()
        want = torch.ones(1, 4)
        if rank == 1:
            want[0, 3] = 0.0  # the padded column receives no gradient
        assert torch.equal(local.grad, want)
        y = ops.reduce_sum(torch.ones(2, requires_grad=True) * (rank + 1))
        assert torch.equal(y.detach(), torch.full((2,), 3.0))
    finally:
        dist.destroy_process_group()


def test_parallel_ops_under_gloo_and_uninitialised():
    from crosslayer_coding_b200.parallel import ops

    assert ops.get_rank() == 0 and ops.get_world_size() == 1 and ops.is_main_process()
    t = torch.ones(2)
    assert ops.all_reduce(t) is None and ops.broadcast(t, 0) is None
    lst = [None]
    ops.all_gather(lst, t)
    assert lst[0] is t
    mp.spawn(_ops_worker, args=(2, _free_port()), nprocs=2, join=True)


def _layers_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from crosslayer_coding_b200.parallel.layers import ColumnParallelLinear, RowParallelLinear

        g = torch.Generator().manual_seed(3)
        d_in, feats, d_out, rows = 6, 21, 5, 7  # 21 features over 2 ranks: shards of 16 with 5 valid on the last rank
        w_col, b_col = torch.randn(feats, d_in, generator=g), torch.randn(feats, generator=g)
        w_row, b_row = torch.randn(d_out, feats, generator=g), torch.randn(d_out, generator=g)
        x = torch.randn(rows, d_in, generator=g)
        col = ColumnParallelLinear(d_in, feats, process_group=dist.group.WORLD)
        row = RowParallelLinear(feats, d_out, process_group=dist.group.WORLD)
        assert col.local_features == 16 and col.valid_features == (16 if rank == 0 else 5)
        lo, n = col.feature_start, col.valid_features
        with torch.no_grad():
            col.weight.zero_(); col.bias_param.zero_(); row.weight.zero_()
            col.weight[:n].copy_(w_col[lo:lo + n]); col.bias_param[:n].copy_(b_col[lo:lo + n])
            row.weight[:, :n].copy_(w_row[:, lo:lo + n]); row.bias_param.copy_(b_row)
        h = col(x)                                   # gathered [rows, feats] on every rank
        y = row(torch.relu(h))                       # split locally, reduced, bias after the reduce
        want_h = x @ w_col.t() + b_col
        want_y = torch.relu(want_h) @ w_row.t() + b_row
        assert h.shape == (rows, feats) and torch.allclose(h, want_h, atol=1e-5)
        assert torch.allclose(y, want_y, atol=1e-5)
        y.sum().backward()
        ref_w = w_col.clone().requires_grad_(True)
        (torch.relu(x @ ref_w.t() + b_col) @ w_row.t() + b_row).sum().backward()
        assert torch.allclose(col.weight.grad[:n], ref_w.grad[lo:lo + n], atol=1e-5)
        assert float(col.weight.grad[n:].abs().sum()) == 0.0  # padding rows receive nothing
    finally:
        dist.destroy_process_group()


def test_standalone_parallel_linear_layers():
    from crosslayer_coding_b200.parallel.layers import ColumnParallelLinear, RowParallelLinear

    col = ColumnParallelLinear(4, 10)
    row = RowParallelLinear(10, 3)
    x = torch.randn(2, 4)
    assert col(x).shape == (2, 10) and row(col(x)).shape == (2, 3) and col.local_features == 10
    mp.spawn(_layers_worker, args=(2, _free_port()), nprocs=2, join=True)


def _full_targets_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from types import SimpleNamespace

        from crosslayer_coding_b200.training.trainer import CLTTrainer

        L, B, d = 3, 8, 4
        rows = B // world
        truth = torch.arange(L * B * d, dtype=torch.float32).view(L, B, d)
        mine = torch.full((L, B, d), -1.0)  # the rows of the other owners are stale on this rank
        mine[:, rank * rows:(rank + 1) * rows] = truth[:, rank * rows:(rank + 1) * rows]
        stub = SimpleNamespace(_target_rows=(rank * rows, rows), world_size=world, process_group=dist.group.WORLD)
        assert torch.equal(CLTTrainer._full_targets(stub, mine), truth)
        stub._target_rows = None  # without the restriction the tensor is passed through
        assert CLTTrainer._full_targets(stub, mine) is mine
    finally:
        dist.destroy_process_group()


def test_evaluation_reassembles_the_owners_target_rows():
    """Tensor-parallel fused runs stage the targets of the owned token rows only; evaluation gathers them again."""
    mp.spawn(_full_targets_worker, args=(2, _free_port()), nprocs=2, join=True)
