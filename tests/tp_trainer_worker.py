"""Worker for the tensor-parallel trainer test (launched with torch.distributed.run, one rank per GPU).

Runs the whole ``CLTTrainer.train()`` loop on the fused engine over a dataset on disk (sharded staging: every rank loads
1/W of the token rows; only the inputs travel to the peers, the targets stay with the token owners), with evaluation and
distributed checkpoints, then checks that the targets which evaluation re-assembles equal the batch of an unsharded store.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from crosslayer_coding_b200 import CLTConfig, TrainingConfig  # noqa: E402
from crosslayer_coding_b200.training.data.local_activation_store import LocalActivationStore  # noqa: E402
from crosslayer_coding_b200.training.trainer import CLTTrainer, _stack_layers  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True)
    ap.add_argument("--log-dir", required=True)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    L, D, F, B = 3, 64, 512, 128
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=D, activation_fn="batchtopk", batchtopk_k=8, clt_dtype="bfloat16")
    tc = TrainingConfig(learning_rate=2e-3, training_steps=16, train_batch_size_tokens=B, activation_path=args.data, activation_dtype="bfloat16",
                        precision="bf16", normalization_method="mean_std", eval_interval=8, checkpoint_interval=8, log_interval=4,
                        engine="fused", aux_loss_factor=1 / 32, dead_feature_window=10, async_checkpoint=True)
    # the process group belongs to this worker (the trainer would otherwise tear its own group down at the end of train(),
    # and the comparison below still needs collectives)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    tr = CLTTrainer(cfg, tc, log_dir=args.log_dir, distributed=True)
    rank, world, dev = tr.rank, tr.world_size, tr.device
    assert tr.engine is not None
    owner_only = getattr(tr, "_target_rows", None) is not None
    tr.train()
    tr.engine.check_status()
    # targets as evaluation sees them against an unsharded store on the same sequence
    common = dict(train_batch_size_tokens=B, device=dev, dtype="bfloat16", rank=rank, world=world, seed=5, sampling_strategy="sequential",
                  normalization_method="mean_std", shard_data=False)
    sharded = LocalActivationStore(args.data, shard_group=dist.group.WORLD, **common)
    sharded.stager.push_only_leading(L)
    plain = LocalActivationStore(args.data, **common)
    layers = list(range(L))
    ok = True
    for _ in range(3):
        xs, ys = next(sharded)
        xp, yp = next(plain)
        full = tr._full_targets(_stack_layers(ys, layers))
        ok = ok and torch.equal(full, _stack_layers(yp, layers)) and torch.equal(_stack_layers(xs, layers), _stack_layers(xp, layers))
    sharded.close()
    plain.close()
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        metrics = json.load(open(os.path.join(args.log_dir, "metrics.json")))
        json.dump({"owner_only": owner_only, "targets_ok": bool(flag.item() == 1.0), "files": sorted(os.listdir(args.log_dir)),
                   "eval": metrics["eval_metrics"][-1], "recon": [v["reconstruction"] for v in metrics["train_losses"]]}, open(args.out, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
