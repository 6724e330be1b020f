"""Worker for the tensor-parallel GPU tests (launched with torch.distributed.run, one rank per GPU).

Builds the same seeded full model on every rank, keeps this rank's feature shard, runs a few fused training
steps on fixed data and writes the per-step losses and the merged (un-sharded) weights from rank 0.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig  # noqa: E402
from crosslayer_coding_b200.training.checkpointing import merge_shards, slice_for_rank  # noqa: E402
from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine  # noqa: E402


def build_full_state(cfg):
    torch.manual_seed(1234)
    full = CrossLayerTranscoder(CLTConfig(**cfg.to_dict()), device="cpu")
    return {k: v.clone() for k, v in full.state_dict().items()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--features", type=int, default=512)
    ap.add_argument("--lam", type=float, default=0.0)
    ap.add_argument("--activation", default="batchtopk")
    ap.add_argument("--tying", default="none")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--clip", type=float, default=0.0)
    ap.add_argument("--affine", action="store_true", help="feature offset / scale of tied decoders")
    ap.add_argument("--dead", action="store_true", help="mark features dead (some on one shard only) and train with the auxiliary loss")
    ap.add_argument("--aux-unfused", action="store_true", help="with --dead under tensor parallelism: take the per-layer PyTorch form of the term")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    L, d, F, B, k = 3, 64, args.features, 128, 8
    t16 = torch.float16 if args.dtype == "float16" else torch.bfloat16
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=args.activation, batchtopk_k=k, topk_k=k, clt_dtype=args.dtype,
                    jumprelu_threshold=0.25, decoder_tying=args.tying, enable_feature_offset=args.affine, enable_feature_scale=args.affine)
    full_state = build_full_state(cfg)
    if args.tying != "none":  # tied decoders start at zero; give them values so that the first steps have a signal
        gen = torch.Generator().manual_seed(99)
        for key in list(full_state):
            if key.startswith("decoder_module.decoders.") and key.endswith(".weight"):
                full_state[key] = (torch.rand(full_state[key].shape, generator=gen) * 0.1 - 0.05).to(full_state[key].dtype)
    if args.affine:
        gen = torch.Generator().manual_seed(123)
        for key in list(full_state):
            if ".feature_offset." in key:
                full_state[key] = (torch.randn(full_state[key].shape, generator=gen) * 0.2).to(full_state[key].dtype)
            if ".feature_scale." in key:
                full_state[key] = (1.0 + torch.randn(full_state[key].shape, generator=gen) * 0.2).to(full_state[key].dtype)
    model = CrossLayerTranscoder(cfg, process_group=group, device=dev)
    model.load_state_dict(slice_for_rank(full_state, rank, world, F) if world > 1 else full_state)
    tc = TrainingConfig(learning_rate=1e-3, training_steps=100, activation_path="unused", precision="fp16" if args.dtype == "float16" else "bf16",
                        sparsity_lambda=args.lam, preactivation_coef=0.0, gradient_clip_val=(args.clip or None), loss_scale_init=1024.0)
    symm = None
    if world > 1:
        from crosslayer_coding_b200.parallel.symm import SymmetricExchange

        symm = SymmetricExchange.create(group, dev, cfg, B)
    eng = FusedBatchTopKEngine(model, tc, B, symm=symm)
    g = torch.Generator().manual_seed(7)
    X = torch.randn(L, B, d, generator=g).to(t16).to(dev)
    A = torch.randn(d, d, generator=g) / d ** 0.5
    Y = (X.float().cpu() @ A).to(t16).to(dev)
    # the selection on the initial weights, as (token, global flat feature index) pairs of all ranks
    eng.encode_select(X)
    n0 = int(eng.ctl[3])
    col = eng.ent_col[:n0].long()
    flat = (col // eng.Fl) * F + model.feature_start + col % eng.Fl
    pairs = torch.stack([eng.ent_tok[:n0].long(), flat], dim=1).cpu()
    if world > 1:
        gathered_pairs = [None] * world
        dist.all_gather_object(gathered_pairs, pairs)
        pairs = torch.cat(gathered_pairs)
    selection = sorted(map(tuple, pairs.tolist()))
    losses, entries, norms = [], [], []
    extra = {}
    if args.dead:
        dead_full = torch.zeros(L, F, dtype=torch.bool)
        dead_full[0, 3:40] = True       # on the first shard only
        dead_full[2, ::5] = True        # spread over every shard
        lo = model.feature_start
        extra = dict(aux_factor=0.5, dead_mask=dead_full[:, lo:lo + model.valid_features].to(dev))
        if args.aux_unfused and world > 1:
            eng.set_dead_count_hint(int(extra["dead_mask"].sum(dim=1).max()), 10 ** 6)  # as if more than k_aux features were dead
    for step in range(args.steps):
        out = eng.train_step(X, Y, step, 1e-3, sparsity_lambda=args.lam, **extra)
        losses.append(float(out.total))
        norms.append(float(out.grad_norm))
        n = out.num_entries.clone().float()
        if world > 1:
            dist.all_reduce(n)
        entries.append(int(n))
    torch.cuda.synchronize()
    eng.check_status()
    # sharded staging: every rank copies 1/W of each batch host->device, the rest arrives over NVLink
    from crosslayer_coding_b200.training.data import InMemoryActivationStore

    pool = torch.randn(4, 2, L, B, d, generator=torch.Generator().manual_seed(11)).bfloat16()
    store = InMemoryActivationStore(pool, dev, loop=True, prefetch=2, shard_group=group)
    staging_ok = True
    for i in range(6):
        inputs, targets = next(store)
        got_x = torch.stack([inputs[l] for l in range(L)]).cpu()
        got_y = torch.stack([targets[l] for l in range(L)]).cpu()
        staging_ok = staging_ok and torch.equal(got_x, pool[i % 4, 0]) and torch.equal(got_y, pool[i % 4, 1])
    # the same through a chunked dataset on disk: rank-sharded native assembly + gather must equal the plain store
    import tempfile

    from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset
    from crosslayer_coding_b200.training.data.local_activation_store import LocalActivationStore

    ds_dir = os.path.join(tempfile.gettempdir(), f"clt_tp_ds_{os.environ.get('MASTER_PORT', '0')}")
    if rank == 0 and not os.path.exists(os.path.join(ds_dir, "metadata.json")):
        write_synthetic_dataset(ds_dir, SyntheticSpec(num_layers=L, d_model=d, dict_size=128, active_mean=4, seed=3),
                                total_tokens=1024, chunk_tokens=256, dtype="bfloat16", device="cpu")
    if world > 1:
        dist.barrier()
    common = dict(train_batch_size_tokens=B, device=dev, dtype="bfloat16", rank=rank, world=world, seed=5, sampling_strategy="random_chunk",
                  normalization_method="mean_std", shard_data=False)
    sharded = LocalActivationStore(ds_dir, shard_group=group, **common)
    plain = LocalActivationStore(ds_dir, **common)
    for i in range(5):
        xs, ys = next(sharded)
        xp, yp = next(plain)
        staging_ok = staging_ok and torch.equal(xs.stacked, xp.stacked) and torch.equal(ys.stacked, yp.stacked)
    sharded.close()
    plain.close()
    flag = torch.tensor([1.0 if staging_ok else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    sd = {k: v.detach().float().cpu() for k, v in model.state_dict().items()}
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, sd)
        merged = merge_shards(gathered, F)
    else:
        merged = sd
    if rank == 0:
        torch.save({"selection": selection, "losses": losses, "entries": entries, "grad_norms": norms, "skipped": float(out.skipped_steps), "state": merged, "world": world, "staging_ok": bool(flag.item() == 1.0),
                    "h2d_bytes_per_rank": store.h2d_bytes_per_rank, "h2d_bytes": store.h2d_bytes_per_batch}, args.out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
