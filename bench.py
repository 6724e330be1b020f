#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the GPT-2-small-shaped cross-layer transcoder
(12 layers, d_model 768, 24576 features per layer = 32x, untied decoders, BatchTopK k=200, 4096-token
batches, bf16) on N GPUs of one node, features tensor-parallel over the GPUs.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29501 \
        bench.py --gpus 2 --steps 20 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same config

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) over steps whose inputs
are already on the device; ``e2e`` is the same metric through the public trainer API with the per-step
host->device copy of the batch from pinned memory and a device->host read of the loss inside the timed region.
Data are synthetic (seeded sparse-dictionary activations), weights are randomly initialised.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

SHAPES = {
    # the headline configuration, and the Llama-3.2-1B-shaped one (16 layers, d_model 2048, 32768 features/layer)
    "gpt2-small": dict(num_layers=12, d_model=768, num_features=24576, k=200, batch=4096, label="GPT-2-small"),
    "llama-3.2-1b": dict(num_layers=16, d_model=2048, num_features=32768, k=200, batch=4096, label="Llama-3.2-1B"),
}
MODEL = dict(SHAPES["gpt2-small"])


def jumprelu_theta() -> float:
    """--activation jumprelu: the threshold that leaves about k of a token's L*F pre-activations active at
    initialisation (encoder rows uniform in +-1/sqrt(F), unit-variance inputs): 0.33 for the GPT-2 shape."""
    import math
    from statistics import NormalDist

    p = MODEL["k"] / (MODEL["num_layers"] * MODEL["num_features"])
    return NormalDist().inv_cdf(1.0 - p) * math.sqrt(MODEL["d_model"] / (3.0 * MODEL["num_features"]))
METRIC = "train tokens/sec (box, device-timed, max over ranks) GPT-2-small CLT 32x BatchTopK"


def metric_name(jr: bool) -> str:
    m = METRIC.replace("GPT-2-small", MODEL["label"])
    if MODEL["label"] != "GPT-2-small":
        m = m.replace("32x", f"{MODEL['num_features'] // MODEL['d_model']}x")
    return m.replace("BatchTopK", "JumpReLU (native thresholds)") if jr else m


def model_name(jr: bool) -> str:
    act = f"JumpReLU theta0={jumprelu_theta():.3f}, sparsity lambda 1e-3" if jr else f"BatchTopK k={MODEL['k']}"
    return (f"{MODEL['label']}-shaped CLT: {MODEL['num_layers']} layers, d_model {MODEL['d_model']}, {MODEL['num_features']} features/layer "
            f"({MODEL['num_features'] // MODEL['d_model']}x), untied decoders, {act}")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--ref-variant", choices=["bf16_params", "autocast_fp32"], default="bf16_params")
    ap.add_argument("--pool", type=int, default=4, help="distinct synthetic batches kept in pinned host memory")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="gpt2-small", help="model shape; gpt2-small is the headline configuration")
    ap.add_argument("--parity-steps", type=int, default=0,
                    help="after the timed loops, train this many further steps over the pool and report the normalised MSE "
                         "on a held-out synthetic batch (key 'parity'); use the same value and --pool for both arms")
    ap.add_argument("--activation", choices=["batchtopk", "jumprelu"], default="batchtopk",
                    help="batchtopk is the headline configuration; jumprelu trains thresholds natively (threshold 0.33: "
                         "about k active features per token on the synthetic data, sparsity penalty on)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report nothing rather than failing the benchmark
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0)),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0)),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0)),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0)),
        }
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = get_reasons(self.h)
                for name, bit in names.items():
                    if bit and mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def setup_dist(n_gpus: int):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    else:
        torch.cuda.set_device(0)
    if world != n_gpus and rank == 0:
        print(f"note: --gpus {n_gpus} but WORLD_SIZE={world}; using WORLD_SIZE", file=sys.stderr)
    return world, rank, local


def heldout_batch(device):
    """One synthetic batch that is in no pool (seed outside the pool's range), on the device: ``[2, L, B, d]`` bf16."""
    import torch

    from crosslayer_coding_b200.activation_generation.synthetic import SparseDictionarySynth, SyntheticSpec

    L, d, B = MODEL["num_layers"], MODEL["d_model"], MODEL["batch"]
    synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=4 * d, active_mean=32.0, seed=1234), device=device)
    synth.fit_norm_stats(8192)
    x, y = synth.sample(B, seed=987654, normalize=True, dtype=torch.bfloat16)
    out = torch.stack([x, y])
    del synth
    return out


def nmse_of(yhat, y) -> float:
    """Mean over layers of MSE / mean_d var_tokens(target), on ``[L, B, d]`` tensors."""
    yf, hf = y.float(), yhat.float()
    mse = ((hf - yf) ** 2).mean(dim=(1, 2))
    var = yf.var(dim=1, unbiased=False).mean(dim=1)
    return float((mse / var).mean())


def make_pool(pool: int, device):
    """``[pool, 2, L, B, d]`` bf16 batches in pinned host memory plus the target std used by the loss."""
    import torch

    from crosslayer_coding_b200.activation_generation.synthetic import SparseDictionarySynth, SyntheticSpec

    L, d, B = MODEL["num_layers"], MODEL["d_model"], MODEL["batch"]
    synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=4 * d, active_mean=32.0, seed=1234), device=device)
    synth.fit_norm_stats(8192)
    host = torch.empty(pool, 2, L, B, d, dtype=torch.bfloat16).pin_memory()
    for i in range(pool):
        x, y = synth.sample(B, seed=1000 + i, normalize=True, dtype=torch.bfloat16)
        host[i, 0].copy_(x)
        host[i, 1].copy_(y)
    torch.cuda.synchronize()
    stats = (synth.mean_tg.float().cpu(), synth.std_tg.float().cpu())
    del synth
    torch.cuda.empty_cache()
    return host, stats


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sync_all(world: int):
    import torch
    import torch.distributed as dist

    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def time_loop(fn, warmup: int, steps: int, world: int, local: int):
    """Device time of ``steps`` calls of ``fn(i)`` after ``warmup`` untimed calls: (ms total max over ranks, clocks)."""
    import torch

    for i in range(warmup):
        fn(i)
    sync_all(world)
    sampler = ClockSampler(local)
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        fn(warmup + i)
    end.record()
    sync_all(world)
    clocks = sampler.stop()
    return max_over_ranks(start.elapsed_time(end), world), clocks


# ----------------------------------------------------------------------------------------------- our arm
def run_ours(args, world, rank, local):
    import torch

    from crosslayer_coding_b200 import CLTConfig, TrainingConfig
    from crosslayer_coding_b200.training.data import InMemoryActivationStore
    from crosslayer_coding_b200.training.trainer import CLTTrainer

    dev = torch.device(f"cuda:{local}")
    L, d, F, k, B = (MODEL[n] for n in ("num_layers", "d_model", "num_features", "k", "batch"))
    host, (mean_tg, std_tg) = make_pool(args.pool, dev)
    jr = args.activation == "jumprelu"
    clt_cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=args.activation, batchtopk_k=k, clt_dtype="bfloat16",
                        jumprelu_threshold=jumprelu_theta())
    total = args.warmup * 2 + args.steps * 2 + 8
    tc = TrainingConfig(
        learning_rate=1e-4, training_steps=max(total, 1000), train_batch_size_tokens=B, precision="bf16",
        activation_path="in-memory", activation_dtype="bfloat16", normalization_method="mean_std",
        sparsity_lambda=(1e-3 if jr else 0.0), sparsity_lambda_schedule="linear", sparsity_lambda_delay_frac=0.0,
        preactivation_coef=0.0, aux_loss_factor=1 / 32, apply_sparsity_penalty_to_batchtopk=False,
        optimizer="adamw", lr_scheduler="linear", eval_interval=10 ** 9, checkpoint_interval=10 ** 9, log_interval=10 ** 9,
        engine="fused",
    )
    shard_group = None
    if world > 1:
        import torch.distributed as dist

        shard_group = dist.group.WORLD  # each rank copies 1/W of a batch over PCIe, the rest arrives over NVLink
    store = InMemoryActivationStore(host, dev, loop=True, prefetch=3 if world > 1 else 2, shard_group=shard_group)
    store.mean_tg = {l: mean_tg[l].to(dev) for l in range(L)}
    store.std_tg = {l: (std_tg[l] + 1e-6).to(dev) for l in range(L)}
    log_dir = tempfile.mkdtemp(prefix="clt_bench_")
    trainer = CLTTrainer(clt_cfg, tc, log_dir=log_dir, device=dev, distributed=world > 1, activation_store=store)
    engine = trainer.engine
    assert engine is not None, "the benchmark requires the fused engine"

    # ---- device-timed: batches resident on the device (151 MB each, larger than L2), cycled
    from crosslayer_coding_b200.training.data.base_store import LayerBatch

    resident = [host[i].to(dev) for i in range(min(args.pool, 3))]
    layers = list(range(L))

    def dev_step(i):
        b = resident[i % len(resident)]
        trainer.train_step(LayerBatch.from_stacked(b[0], layers), LayerBatch.from_stacked(b[1], layers), i)

    launches0 = engine.kernel_launches
    ms, clocks = time_loop(dev_step, args.warmup, args.steps, world, local)
    launches = (engine.kernel_launches - launches0) * args.steps // (args.warmup + args.steps)
    engine.check_status()
    del resident

    # ---- end to end through the trainer API: pinned host batch -> device every step, loss read back
    step_box = [args.warmup + args.steps]
    losses = []

    # every step's loss is read back (4 bytes, device -> pinned host); the read of step i is collected after
    # step i + 1 has been queued, so the host never idles the GPU while it waits for a scalar
    loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ready = [torch.cuda.Event() for _ in range(2)]
    pending = []

    def collect():
        slot = pending.pop(0)
        loss_ready[slot].synchronize()
        losses.append(float(loss_host[slot][0]))

    def e2e_step(i):
        inputs, targets = next(store)
        parts = trainer.train_step(inputs, targets, step_box[0])
        step_box[0] += 1
        slot = i % 2
        loss_host[slot].copy_(parts["total"].detach().float().reshape(1), non_blocking=True)
        loss_ready[slot].record()
        pending.append(slot)
        if len(pending) > 1:
            collect()

    for i in range(args.warmup):
        e2e_step(i)
    while pending:
        collect()
    sync_all(world)
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    while pending:
        collect()
    sync_all(world)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    engine.check_status()

    parity = None
    if args.parity_steps > 0:
        for i in range(args.parity_steps):
            inputs, targets = next(store)
            trainer.train_step(inputs, targets, step_box[0])
            step_box[0] += 1
        held = heldout_batch(dev)
        with torch.no_grad():
            yhat = engine.forward(held[0], held[1])
        engine.check_status()
        parity = {"steps_trained": step_box[0], "nmse_heldout": nmse_of(yhat, held[1]), "pool_batches": args.pool}

    value = B * args.steps / (ms / 1e3)
    e2e_value = B * args.steps / (e2e_ms / 1e3)
    return {
        "metric": metric_name(jr),
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded sparse-dictionary activations, random-init weights)",
        "config": {
            "model": model_name(jr),
            "global_batch": B, "seq_len": 1, "parallelism": f"tp{world}",
            "optimizer": "AdamW, fp32 moments, bf16 weights", "loss": "reconstruction + AuxK factor 1/32 (no dead features yet)",
            "l2": "per-step inputs (151 MB) and streamed weights (3.4 GB) exceed the 126 MB L2; 3 device batches cycled",
        },
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": int(store.h2d_bytes_per_batch), "d2h_bytes_per_step": 4 * world,
                "h2d_bytes_per_step_per_rank": int(store.h2d_bytes_per_rank),
                "staging": ("pinned host ring -> side-stream copy of this rank's 1/W token rows -> "
                            + ("copy-engine push into every peer's symmetric-memory slot over NVLink" if getattr(store.stager, "push", False)
                               else "NVLink all-gather")) if world > 1 else "pinned host ring -> side-stream copy"},
        "gpu_launches": int(launches),
        "final_loss": losses[-1] if losses else None,
        "parity": parity,
        "impl": "ours",
    }


# ------------------------------------------------------------------------------------------ reference arm
def run_reference(args, world, rank, local):
    import torch
    import torch.distributed as dist

    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "clt")):
        return {"impl": "reference", "unavailable": "baseline/_ref is missing (reference not installed)"}
    sys.path.insert(0, ref_root)
    try:
        from clt.config import CLTConfig as RefCLTConfig, TrainingConfig as RefTrainingConfig
        from clt.models.clt import CrossLayerTranscoder as RefCLT
        from clt.training.distributed_utils import average_shared_parameter_grads
        from clt.training.losses import LossManager as RefLossManager
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"}
    trainer_note = None
    try:
        import clt.training.trainer  # noqa: F401
    except Exception as exc:  # noqa: BLE001
        trainer_note = f"{type(exc).__name__}: {exc}"

    dev = torch.device(f"cuda:{local}")
    L, d, F, k, B = (MODEL[n] for n in ("num_layers", "d_model", "num_features", "k", "batch"))
    host, (mean_tg, std_tg) = make_pool(args.pool, dev)
    bf16_params = args.ref_variant == "bf16_params"
    jr = args.activation == "jumprelu"
    cfg = RefCLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=args.activation, batchtopk_k=k,
                       jumprelu_threshold=jumprelu_theta(), clt_dtype="bfloat16" if bf16_params else None)
    tc = RefTrainingConfig(
        learning_rate=1e-4, training_steps=1000, train_batch_size_tokens=B, precision="bf16",
        activation_path="in-memory", activation_dtype="bfloat16", normalization_method="mean_std",
        sparsity_lambda=(1e-3 if jr else 0.0), sparsity_lambda_schedule="linear", sparsity_lambda_delay_frac=0.0,
        preactivation_coef=0, aux_loss_factor=1 / 32, apply_sparsity_penalty_to_batchtopk=False,
        optimizer="adamw", lr_scheduler="linear",
    )
    torch.manual_seed(tc.seed + rank)
    group = dist.group.WORLD if world > 1 else None
    model = RefCLT(cfg, process_group=group, device=dev)
    opt = torch.optim.AdamW(model.parameters(), lr=tc.learning_rate)
    sched = torch.optim.lr_scheduler.LinearLR(opt, start_factor=1.0, end_factor=0.1, total_iters=tc.training_steps)
    loss_mgr = RefLossManager(tc, mean_tg={l: mean_tg[l].to(dev) for l in range(L)},
                              std_tg={l: (std_tg[l] + 1e-6).to(dev) for l in range(L)}, clt_config=cfg)
    scaler = torch.amp.GradScaler("cuda", enabled=False)
    since_fired = torch.zeros(L, F, dtype=torch.long, device=dev)

    def step_fn(inputs, targets, step):
        """The reference trainer's step (clt/training/trainer.py:661-810) on the reference's own model and losses."""
        opt.zero_grad(set_to_none=True)
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16, enabled=True):
            acts = model.get_feature_activations(inputs)
            loss, loss_dict = loss_mgr.compute_total_loss(
                model, inputs, targets, step, tc.training_steps, precomputed_activations=acts,
                dead_neuron_mask=(since_fired > tc.dead_feature_window),
            )
        with torch.no_grad():
            for l, a in acts.items():
                fired = (a.detach() > 1e-6).any(dim=0)
                since_fired[l] += 1
                since_fired[l][fired] = 0
        scaler.scale(loss).backward()
        scaler.unscale_(opt)
        if world > 1:
            average_shared_parameter_grads(model, world)
        scaler.step(opt)
        scaler.update()
        if hasattr(model, "decoder_module") and hasattr(model.decoder_module, "_cached_decoder_norms"):
            model.decoder_module._cached_decoder_norms = None
        if world > 1:
            dist.all_reduce(since_fired, op=dist.ReduceOp.MIN, group=group)
        sched.step()
        return loss_dict

    resident = [host[i].to(dev) for i in range(min(args.pool, 3))]

    def as_dicts(b):
        return {l: b[0, l] for l in range(L)}, {l: b[1, l] for l in range(L)}

    def dev_step(i):
        x, y = as_dicts(resident[i % len(resident)])
        step_fn(x, y, i)

    ms, clocks = time_loop(dev_step, args.warmup, args.steps, world, local)
    del resident
    stage = [torch.empty_like(host[0], device=dev) for _ in range(2)]
    losses = []

    def e2e_step(i):
        buf = stage[i % 2]
        buf.copy_(host[i % args.pool], non_blocking=True)
        x, y = as_dicts(buf)
        ld = step_fn(x, y, args.warmup + args.steps + i)
        losses.append(float(ld["total"]))

    for i in range(min(args.warmup, 2)):
        e2e_step(i)
    sync_all(world)
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    sync_all(world)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    parity = None
    if args.parity_steps > 0:
        done = args.warmup + args.steps + min(args.warmup, 2) + args.steps
        for i in range(args.parity_steps):
            buf = stage[i % 2]
            buf.copy_(host[i % args.pool], non_blocking=True)
            x, y = as_dicts(buf)
            step_fn(x, y, done + i)
        held = heldout_batch(dev)
        with torch.no_grad(), torch.autocast(device_type="cuda", dtype=torch.bfloat16, enabled=True):
            out = model({l: held[0, l] for l in range(L)})
        yhat = torch.stack([out[l].float() for l in range(L)])
        parity = {"steps_trained": done + args.parity_steps, "nmse_heldout": nmse_of(yhat, held[1]), "pool_batches": args.pool}
    return {
        "metric": metric_name(jr),
        "value": B * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded sparse-dictionary activations, random-init weights)",
        "config": {
            "model": model_name(jr),
            "global_batch": B, "seq_len": 1, "parallelism": f"tp{world}", "variant": args.ref_variant,
            "path": "reference CrossLayerTranscoder + LossManager + average_shared_parameter_grads driven through the step "
                    "sequence of clt/training/trainer.py:661-810" + (f" (CLTTrainer itself is not importable: {trainer_note})" if trainer_note else ""),
        },
        "clocks": clocks,
        "e2e": {"value": B * args.steps / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": int(host[0].numel() * 2), "d2h_bytes_per_step": 20},
        "gpu_launches": 0,
        "final_loss": losses[-1] if losses else None,
        "parity": parity,
        "impl": "reference",
    }


def main():
    args = parse_args()
    MODEL.clear()
    MODEL.update(SHAPES[args.shape])
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return 0
    world, rank, local = setup_dist(args.gpus)
    try:
        if args.impl == "reference":
            try:
                result = run_reference(args, world, rank, local)
            except Exception as exc:  # noqa: BLE001 - the reference arm must never take the benchmark down
                result = {"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {str(exc)[:300]}"}
        else:
            result = run_ours(args, world, rank, local)
        if rank == 0:
            print(json.dumps(result))
    finally:
        if world > 1:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
