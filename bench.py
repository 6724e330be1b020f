#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the GPT-2-small-shaped cross-layer transcoder
(12 layers, d_model 768, 24576 features per layer = 32x, untied decoders, BatchTopK k=200, 4096-token
batches, bf16) on N GPUs of one node, features tensor-parallel over the GPUs.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29501 \
        bench.py --gpus 2 --steps 20 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same config

Variants of the same measurement: ``--shape pythia-70m|llama-3.2-1b``, ``--decoder-tying``, ``--precision fp16``, ``--activation
jumprelu``, ``--dead-frac`` (AuxK in every step), ``--store local`` (HDF5 chunks on disk), ``--parity-steps`` (held-out normalised
MSE after further training, optionally a fresh batch per step and a curve), ``--stochastic-rounding``; other measurements:
``--mode inference|convert|decode-reduce``.

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
    # the headline configuration; the Pythia-70m-shaped one (tied decoders, fp16 with loss scaling, 8192-token batches);
    # the Llama-3.2-1B-shaped one (16 layers, d_model 2048, 32768 features/layer, JumpReLU)
    "gpt2-small": dict(num_layers=12, d_model=768, num_features=24576, k=200, batch=4096, label="GPT-2-small", dict_mult=4, active=32.0),
    "pythia-70m": dict(num_layers=6, d_model=512, num_features=32768, k=200, batch=8192, label="Pythia-70m", dict_mult=4, active=24.0),
    "llama-3.2-1b": dict(num_layers=16, d_model=2048, num_features=32768, k=200, batch=4096, label="Llama-3.2-1B", dict_mult=4, active=48.0),
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


TYING_LABEL = {"none": "untied decoders", "per_source": "per-source tied decoders", "per_target": "per-target tied decoders"}


def model_name(jr: bool) -> str:
    act = f"JumpReLU theta0={jumprelu_theta():.3f}, sparsity lambda 1e-3" if jr else f"BatchTopK k={MODEL['k']}"
    return (f"{MODEL['label']}-shaped CLT: {MODEL['num_layers']} layers, d_model {MODEL['d_model']}, {MODEL['num_features']} features/layer "
            f"({MODEL['num_features'] // MODEL['d_model']}x), {TYING_LABEL[MODEL.get('tying', 'none')]}, {act}")


def config_block(args, world: int, jr: bool) -> dict:
    """The ``config`` entry of the result line: the same keys and values in both arms (what was measured, not how)."""
    prec = args.precision
    return {
        "model": model_name(jr),
        "global_batch": MODEL["batch"], "seq_len": 1, "parallelism": f"tp{world}",
        "optimizer": f"AdamW, fp32 moments, {prec} compute" + (", dynamic loss scaling" if prec == "fp16" else ""),
        "loss": "reconstruction" + (" + tanh sparsity penalty (lambda 1e-3, linear warm-up)" if jr else "") + " + AuxK factor 1/32"
                + (f" ({args.dead_frac:.0%} of the features marked dead)" if args.dead_frac > 0 else " (no dead features yet)"),
        "l2": "per-step inputs and streamed weights exceed the 126 MB L2; 3 device batches cycled",
    }


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
    ap.add_argument("--parity-fresh", action="store_true",
                    help="--parity-steps draws a fresh synthetic batch every step (seeded by the step, the same stream in both arms) "
                         "instead of cycling the pool: a convergence run")
    ap.add_argument("--parity-log-every", type=int, default=0, help="record the held-out normalised MSE every this many parity steps (key 'parity.curve')")
    ap.add_argument("--stochastic-rounding", action="store_true",
                    help="our arm: round the updated 16-bit weights stochastically (TrainingConfig.enable_stochastic_rounding); small "
                         "late-schedule updates are otherwise lost to round-to-nearest")
    ap.add_argument("--decoder-tying", choices=["none", "per_source", "per_target"], default="none")
    ap.add_argument("--precision", choices=["bf16", "fp16"], default="bf16", help="fp16: fp16 weights / activations with dynamic loss scaling")
    ap.add_argument("--batch", type=int, default=None, help="tokens per batch (default: the shape's)")
    ap.add_argument("--dead-frac", type=float, default=0.0,
                    help="mark this fraction of every layer's features dead before the run, so that the AuxK term is part of every timed step")
    ap.add_argument("--store", choices=["memory", "local"], default="memory",
                    help="end-to-end data source: batches in pinned host memory, or a bf16 HDF5 dataset on disk read through LocalActivationStore")
    ap.add_argument("--mode", choices=["train", "inference", "convert", "decode-reduce"], default="train",
                    help="train: the headline metric; inference / convert / decode-reduce: the sweeps of the inference and conversion configuration")
    ap.add_argument("--convert-tokens", type=int, default=2_000_000, help="--mode convert: tokens used for the threshold estimation")
    ap.add_argument("--activation", choices=["batchtopk", "jumprelu"], default="batchtopk",
                    help="batchtopk is the headline configuration; jumprelu trains thresholds natively (threshold 0.33: "
                         "about k active features per token on the synthetic data, sparsity penalty on)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, active: bool = True):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.nv = None
        if not active:
            return
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
    synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=MODEL["dict_mult"] * d, active_mean=MODEL["active"], seed=1234), device=device)
    synth.fit_norm_stats(8192)
    x, y = synth.sample(B, seed=987654, normalize=True, dtype=torch.bfloat16)
    out = torch.stack([x, y])
    del synth
    return out


class FreshBatches:
    """The seeded synthetic stream, one new ``[2, L, B, d]`` batch per call, generated on the device (convergence runs)."""

    def __init__(self, device):
        from crosslayer_coding_b200.activation_generation.synthetic import SparseDictionarySynth, SyntheticSpec

        L, d = MODEL["num_layers"], MODEL["d_model"]
        self.synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=MODEL["dict_mult"] * d, active_mean=MODEL["active"], seed=1234), device=device)
        self.synth.fit_norm_stats(8192)

    def __call__(self, i: int):
        import torch

        t16 = torch.float16 if MODEL.get("precision") == "fp16" else torch.bfloat16
        x, y = self.synth.sample(MODEL["batch"], seed=100000 + i, normalize=True, dtype=t16)
        return torch.stack([x, y])


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
    synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=MODEL["dict_mult"] * d, active_mean=MODEL["active"], seed=1234), device=device)
    synth.fit_norm_stats(8192)
    t16 = torch.float16 if MODEL.get("precision") == "fp16" else torch.bfloat16
    host = torch.empty(pool, 2, L, B, d, dtype=t16).pin_memory()
    for i in range(pool):
        x, y = synth.sample(B, seed=1000 + i, normalize=True, dtype=t16)
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
    # rank 0 samples its own GPU; NVML queries from every rank at once take the driver's lock often enough to show in a
    # timed region of a few tens of milliseconds.  NVML is initialised before the barrier: a rank that enters the timed
    # region late keeps the others waiting at their first exchange.
    sampler = ClockSampler(local, active=int(os.environ.get("RANK", "0")) == 0)
    sync_all(world)
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        fn(warmup + i)
    end.record()
    sync_all(world)
    clocks = sampler.stop()
    return max_over_ranks(start.elapsed_time(end), world), clocks


DEAD_WINDOW = 10 ** 6  # nothing dies of its own during a benchmark run; --dead-frac marks features dead explicitly


def tying_needs_init(args) -> bool:
    return args.decoder_tying != "none"


def make_local_store(args, dev, world, rank, shard_group):
    """--store local: the seeded synthetic stream written as bf16 HDF5 chunks (raw values + norm_stats.json) and read back
    through LocalActivationStore: chunk files -> native threaded row gather into the pinned ring -> side-stream copy of
    this rank's rows -> push to the peers; normalisation is applied by the store."""
    import torch
    import torch.distributed as dist

    from crosslayer_coding_b200.activation_generation.synthetic import SyntheticSpec, write_synthetic_dataset
    from crosslayer_coding_b200.training.data.local_activation_store import LocalActivationStore

    L, d, B = MODEL["num_layers"], MODEL["d_model"], MODEL["batch"]
    chunk = 4 * B
    tokens = ((args.warmup + args.steps + 6) * B + chunk - 1) // chunk * chunk
    root = os.path.join(tempfile.gettempdir(), f"clt_bench_ds_{MODEL['label']}_{B}_{tokens}")
    if rank == 0 and not os.path.exists(os.path.join(root, "metadata.json")):
        write_synthetic_dataset(root, SyntheticSpec(num_layers=L, d_model=d, dict_size=MODEL["dict_mult"] * d, active_mean=MODEL["active"], seed=1234),
                                total_tokens=tokens, chunk_tokens=chunk, dtype="bfloat16", device=str(dev))
    if world > 1:
        dist.barrier()
    store = LocalActivationStore(root, train_batch_size_tokens=B, device=dev, dtype="float16" if args.precision == "fp16" else "bfloat16",
                                 rank=rank, world=world, seed=5, sampling_strategy="sequential", normalization_method="mean_std",
                                 shard_data=False, shard_group=shard_group, prefetch_batches=3)
    note = f"LocalActivationStore over {tokens} tokens in bf16 HDF5 chunks of {chunk} tokens, normalised by the store"
    return store, note


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
    fp16 = args.precision == "fp16"
    clt_cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=args.activation, batchtopk_k=k,
                        clt_dtype="float16" if fp16 else "bfloat16", jumprelu_threshold=jumprelu_theta(), decoder_tying=args.decoder_tying)
    total = args.warmup * 2 + args.steps * 2 + 8 + args.parity_steps
    tc = TrainingConfig(
        learning_rate=1e-4, training_steps=max(total, 1000), train_batch_size_tokens=B, precision=args.precision,
        activation_path="in-memory", activation_dtype="float16" if fp16 else "bfloat16", normalization_method="mean_std",
        sparsity_lambda=(1e-3 if jr else 0.0), sparsity_lambda_schedule="linear", sparsity_lambda_delay_frac=0.0,
        preactivation_coef=0.0, aux_loss_factor=1 / 32, apply_sparsity_penalty_to_batchtopk=False,
        optimizer="adamw", lr_scheduler="linear", eval_interval=10 ** 9, checkpoint_interval=10 ** 9, log_interval=10 ** 9,
        engine="fused", dead_feature_window=DEAD_WINDOW, enable_stochastic_rounding=bool(args.stochastic_rounding),
    )
    shard_group = None
    if world > 1:
        import torch.distributed as dist

        shard_group = dist.group.WORLD  # each rank copies 1/W of a batch over PCIe, the rest arrives over NVLink
    store_note = None
    if args.store == "local":
        store, store_note = make_local_store(args, dev, world, rank, shard_group)
    else:
        store = InMemoryActivationStore(host, dev, loop=True, prefetch=3 if world > 1 else 2, shard_group=shard_group)
        store.mean_tg = {l: mean_tg[l].to(dev) for l in range(L)}
        store.std_tg = {l: (std_tg[l] + 1e-6).to(dev) for l in range(L)}
    log_dir = tempfile.mkdtemp(prefix="clt_bench_")
    trainer = CLTTrainer(clt_cfg, tc, log_dir=log_dir, device=dev, distributed=world > 1, activation_store=store)
    engine = trainer.engine
    assert engine is not None, "the benchmark requires the fused engine"
    if tying_needs_init(args):
        with torch.no_grad():  # tied decoders start at zero (reference decoder.py:80-86): nothing would be selected for the decode
            for w in trainer.model.dec_weight:
                w.uniform_(-1.0 / (L * d) ** 0.5, 1.0 / (L * d) ** 0.5)
    if args.dead_frac > 0:
        # every n-th feature of every layer counts as dead from the start: AuxK is part of every timed step
        stride = max(1, int(round(1.0 / args.dead_frac)))
        engine.dead_counter.view(L, engine.Fl)[:, ::stride] = DEAD_WINDOW + 1

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
        held = heldout_batch(dev)
        fresh = FreshBatches(dev) if args.parity_fresh else None
        curve = []

        def heldout_nmse():
            with torch.no_grad():
                yhat = engine.forward(held[0].to(engine.t16), held[1].to(engine.t16))
            return nmse_of(yhat, held[1])

        for i in range(args.parity_steps):
            if fresh is not None:
                b = fresh(i)
                inputs, targets = LayerBatch.from_stacked(b[0], layers), LayerBatch.from_stacked(b[1], layers)
            else:
                inputs, targets = next(store)
            trainer.train_step(inputs, targets, step_box[0])
            step_box[0] += 1
            if args.parity_log_every and (i + 1) % args.parity_log_every == 0:
                curve.append([i + 1, round(heldout_nmse(), 5)])
        engine.check_status()
        parity = {"steps_trained": step_box[0], "nmse_heldout": heldout_nmse(), "pool_batches": args.pool,
                  "data": "fresh batch per step" if fresh is not None else "pool cycled", "curve": curve}

    value = B * args.steps / (ms / 1e3)
    e2e_value = B * args.steps / (e2e_ms / 1e3)
    return {
        "metric": metric_name(jr),
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": args.precision, "data": "synthetic (seeded sparse-dictionary activations, random-init weights)",
        "config": config_block(args, world, jr),
        "arm": {"engine": "fused sm_100a step (crosslayer_coding_b200.training.fused_engine)", "weights": f"{args.precision} parameters, fp32 Adam moments",
                "e2e_store": store_note or "InMemoryActivationStore (pinned host pool)", "skipped_steps": int(engine.step_ctl[7].view(torch.int32))},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": int(store.h2d_bytes_per_batch), "d2h_bytes_per_step": 4 * world,
                "h2d_bytes_per_step_per_rank": int(getattr(store, "h2d_bytes_per_rank", None) or store.stager.h2d_bytes_per_rank),
                "staging": ("pinned host ring -> side-stream copy of this rank's 1/W token rows -> "
                            + ("copy-engine push into every peer's symmetric-memory slot over NVLink" if getattr(getattr(store, "stager", None), "push", False)
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
    fp16 = args.precision == "fp16"
    # fp16 in the reference: fp32 parameters under fp16 autocast with a GradScaler (its documented mode; GradScaler refuses fp16 parameters)
    bf16_params = args.ref_variant == "bf16_params" and not fp16
    jr = args.activation == "jumprelu"
    cfg = RefCLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=args.activation, batchtopk_k=k,
                       jumprelu_threshold=jumprelu_theta(), clt_dtype="bfloat16" if bf16_params else None, decoder_tying=args.decoder_tying)
    tc = RefTrainingConfig(
        learning_rate=1e-4, training_steps=max(args.warmup * 2 + args.steps * 2 + 8 + args.parity_steps, 1000), train_batch_size_tokens=B, precision=args.precision,
        activation_path="in-memory", activation_dtype="float16" if fp16 else "bfloat16", normalization_method="mean_std",
        sparsity_lambda=(1e-3 if jr else 0.0), sparsity_lambda_schedule="linear", sparsity_lambda_delay_frac=0.0,
        preactivation_coef=0, aux_loss_factor=1 / 32, apply_sparsity_penalty_to_batchtopk=False,
        optimizer="adamw", lr_scheduler="linear", dead_feature_window=DEAD_WINDOW,
    )
    torch.manual_seed(tc.seed + rank)
    group = dist.group.WORLD if world > 1 else None
    model = RefCLT(cfg, process_group=group, device=dev)
    opt = torch.optim.AdamW(model.parameters(), lr=tc.learning_rate)
    sched = torch.optim.lr_scheduler.LinearLR(opt, start_factor=1.0, end_factor=0.1, total_iters=tc.training_steps)
    loss_mgr = RefLossManager(tc, mean_tg={l: mean_tg[l].to(dev) for l in range(L)},
                              std_tg={l: (std_tg[l] + 1e-6).to(dev) for l in range(L)}, clt_config=cfg)
    scaler = torch.amp.GradScaler("cuda", enabled=fp16)
    amp_dtype = torch.float16 if fp16 else torch.bfloat16
    since_fired = torch.zeros(L, F, dtype=torch.long, device=dev)
    if tying_needs_init(args):
        with torch.no_grad():  # same start as the other arm: tied decoders would otherwise be all zero
            for name, prm in model.named_parameters():
                if "decoder_module.decoders" in name and name.endswith("weight"):
                    prm.uniform_(-1.0 / (L * d) ** 0.5, 1.0 / (L * d) ** 0.5)
    if args.dead_frac > 0:
        since_fired[:, ::max(1, int(round(1.0 / args.dead_frac)))] = DEAD_WINDOW + 1

    def step_fn(inputs, targets, step):
        """The reference trainer's step (clt/training/trainer.py:661-810) on the reference's own model and losses."""
        opt.zero_grad(set_to_none=True)
        with torch.autocast(device_type="cuda", dtype=amp_dtype, enabled=True):
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
        held = heldout_batch(dev)
        fresh = FreshBatches(dev) if args.parity_fresh else None
        curve = []

        def heldout_nmse():
            with torch.no_grad(), torch.autocast(device_type="cuda", dtype=amp_dtype, enabled=True):
                out = model({l: held[0, l] for l in range(L)})
            return nmse_of(torch.stack([out[l].float() for l in range(L)]), held[1])

        for i in range(args.parity_steps):
            if fresh is not None:
                buf = fresh(i)
            else:
                buf = stage[i % 2]
                buf.copy_(host[i % args.pool], non_blocking=True)
            x, y = as_dicts(buf)
            step_fn(x, y, done + i)
            if args.parity_log_every and (i + 1) % args.parity_log_every == 0:
                curve.append([i + 1, round(heldout_nmse(), 5)])
        parity = {"steps_trained": done + args.parity_steps, "nmse_heldout": heldout_nmse(), "pool_batches": args.pool,
                  "data": "fresh batch per step" if fresh is not None else "pool cycled", "curve": curve}
    return {
        "metric": metric_name(jr),
        "value": B * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": args.precision, "data": "synthetic (seeded sparse-dictionary activations, random-init weights)",
        "config": config_block(args, world, jr),
        "arm": {"variant": ("fp32 parameters, fp16 autocast, GradScaler" if fp16 else args.ref_variant),
                "path": "reference CrossLayerTranscoder + LossManager + average_shared_parameter_grads driven through the step "
                        "sequence of clt/training/trainer.py:661-810" + (f" (CLTTrainer itself is not importable: {trainer_note})" if trainer_note else "")},
        "clocks": clocks,
        "e2e": {"value": B * args.steps / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": int(host[0].numel() * 2), "d2h_bytes_per_step": 20},
        "gpu_launches": 0,
        "final_loss": losses[-1] if losses else None,
        "parity": parity,
        "impl": "reference",
    }



# ------------------------------------------------------------------------------------- inference / conversion sweeps
def _event_ms(fn, warmup: int, iters: int) -> float:
    """Mean device time of ``fn()`` over ``iters`` calls after ``warmup`` calls (CUDA events, synchronised both sides)."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def _synth(device):
    from crosslayer_coding_b200.activation_generation.synthetic import SparseDictionarySynth, SyntheticSpec

    L, d = MODEL["num_layers"], MODEL["d_model"]
    synth = SparseDictionarySynth(SyntheticSpec(num_layers=L, d_model=d, dict_size=MODEL["dict_mult"] * d, active_mean=MODEL["active"], seed=1234), device=device)
    synth.fit_norm_stats(8192)
    return synth


def _reference_model(args, dev, k, activation="batchtopk"):
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "clt")):
        return None, "baseline/_ref is missing (reference not installed)"
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    try:
        import torch
        from clt.config import CLTConfig as RefCLTConfig
        from clt.models.clt import CrossLayerTranscoder as RefCLT
    except Exception as exc:  # noqa: BLE001
        return None, f"reference import failed: {type(exc).__name__}: {exc}"
    L, d, F = (MODEL[n] for n in ("num_layers", "d_model", "num_features"))
    cfg = RefCLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=activation, batchtopk_k=k, clt_dtype="bfloat16")
    torch.manual_seed(42)
    return RefCLT(cfg, process_group=None, device=dev), None


def run_inference_sweep(args, world, rank, local):
    """Encode + decode throughput (tokens/s) for batches of 512 / 4096 / 32768 tokens and k in {32, 200, 1024}: the sparse
    forward of this framework, or ``model(inputs)`` of the reference under bf16 autocast."""
    import torch

    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder
    from crosslayer_coding_b200.models.sparse_forward import SparseForward

    dev = torch.device(f"cuda:{local}")
    L, d, F = (MODEL[n] for n in ("num_layers", "d_model", "num_features"))
    synth = _synth(dev)
    sweep = []
    ours = args.impl == "ours"
    model = None
    for B in (512, 4096, 32768):
        x, _ = synth.sample(B, seed=77, normalize=True, dtype=torch.bfloat16)   # [L, B, d], larger than L2 from 4096 tokens on
        for k in (32, 200, 1024):
            cell = {"batch": B, "k": k}
            try:
                if ours:
                    if model is None:
                        torch.manual_seed(42)
                        model = CrossLayerTranscoder(CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=k,
                                                               clt_dtype="bfloat16"), device=dev)
                    model.config.batchtopk_k = k
                    sf = SparseForward(model, B, max_active_per_token=k)
                    ms = _event_ms(lambda: sf.reconstruct(x), 3, 10 if B < 32768 else 4)
                    sf.check_status()
                    del sf
                else:
                    if model is None:
                        model, why = _reference_model(args, dev, k)
                        if model is None:
                            return {"impl": "reference", "unavailable": why}
                    model.config.batchtopk_k = k
                    need_gb = 3 * B * L * F * 2 / 1e9
                    if need_gb > 120:
                        cell["skipped"] = f"the reference's dense [B, L*F] temporaries would need about {need_gb:.0f} GB"
                        sweep.append(cell)
                        continue
                    inputs = {l: x[l] for l in range(L)}

                    def ref_forward():
                        with torch.no_grad(), torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                            model(inputs)

                    ms = _event_ms(ref_forward, 2, 5 if B < 32768 else 2)
                cell.update(ms=ms, tokens_per_s=B / ms * 1e3)
            except torch.OutOfMemoryError:
                cell["skipped"] = "out of memory"
                torch.cuda.empty_cache()
            sweep.append(cell)
        del x
        torch.cuda.empty_cache()
    head = next((c for c in sweep if c["batch"] == 4096 and c["k"] == 200 and "tokens_per_s" in c), None)
    return {"metric": f"inference encode+decode tokens/sec, {MODEL['label']}-shaped CLT 32x BatchTopK (sweep over batch and k)",
            "value": head["tokens_per_s"] if head else None, "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded sparse-dictionary activations, random-init weights)", "sweep": sweep, "impl": args.impl,
            "config": {"model": model_name(False), "mode": "inference", "headline_cell": "batch 4096, k 200"}}


def run_convert(args, world, rank, local):
    """BatchTopK -> JumpReLU on the random-init model: threshold estimation over ``--convert-tokens`` seeded tokens and the
    layer-wise L0 calibration; wall time on the device and the L0 error per layer against the original model."""
    import torch

    from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder
    from crosslayer_coding_b200.conversion import calibrate_layerwise_theta, layer_l0, quick_l0_check

    dev = torch.device(f"cuda:{local}")
    L, d, F, k, B = (MODEL[n] for n in ("num_layers", "d_model", "num_features", "k", "batch"))
    synth = _synth(dev)
    n_batches = max(1, args.convert_tokens // B)

    def batches():
        for i in range(n_batches):
            x, y = synth.sample(B, seed=5000 + i, normalize=True, dtype=torch.bfloat16)
            yield {l: x[l] for l in range(L)}, {l: y[l] for l in range(L)}

    xc, _ = synth.sample(B, seed=4999, normalize=True, dtype=torch.bfloat16)
    calib = {l: xc[l] for l in range(L)}
    if args.impl == "ours":
        torch.manual_seed(42)
        model = CrossLayerTranscoder(CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=k, clt_dtype="bfloat16"), device=dev)
        target = layer_l0(model, calib)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        model.estimate_theta_posthoc(batches(), num_batches=n_batches)
        torch.cuda.synchronize()
        t_est = time.perf_counter() - t0
        before = quick_l0_check(model, calib, num_tokens=B, seed=0)
        t0 = time.perf_counter()
        scales = calibrate_layerwise_theta(model, calib, target, tolerance=0.5)
        torch.cuda.synchronize()
        t_cal = time.perf_counter() - t0
        after = quick_l0_check(model, calib, num_tokens=B, seed=0)
        err = {l: after[l] - target[l] for l in target}
        extra = {"calibration_s": t_cal, "l0_error_after_calibration": err, "l0_error_before_calibration": {l: before[l] - target[l] for l in target},
                 "scales": scales}
    else:
        model, why = _reference_model(args, dev, k)
        if model is None:
            return {"impl": "reference", "unavailable": why}
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
            model.estimate_theta_posthoc(batches(), num_batches=n_batches)
        torch.cuda.synchronize()
        t_est = time.perf_counter() - t0
        extra = {"calibration_s": None, "note": "the reference's layer-wise calibration lives in its conversion script, outside the installed package"}
    tokens = n_batches * B
    return {"metric": f"BatchTopK->JumpReLU conversion, {MODEL['label']}-shaped CLT: threshold estimation tokens/sec over {tokens} seeded tokens",
            "value": tokens / t_est, "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "estimation_s": t_est,
            "data": "synthetic (seeded sparse-dictionary activations, random-init weights)", "impl": args.impl, **extra,
            "config": {"model": model_name(False), "mode": "convert", "tokens": tokens, "batch": B}}


def run_decode_reduce(args, world, rank, local):
    """Stand-alone sweep of the fused sparse decode -> cross-rank reduce (decode kernel pushing partial rows into the owners'
    staging slots over NVLink, owner reduce with the loss epilogue, gradient-seed all-gather by push) over the density of the
    active features, against dense decoder GEMMs (cuBLAS) with one NCCL all-reduce per (source, target) pair, which is the
    reference's row-parallel path (clt/models/parallel.py:363-383)."""
    import torch
    import torch.distributed as dist

    from crosslayer_coding_b200.ops import ext as ext_mod
    from crosslayer_coding_b200.parallel.symm import SymmetricExchange

    if world < 2:
        return {"impl": args.impl, "unavailable": "decode-reduce needs at least 2 GPUs (launch with torch.distributed.run)"}
    dev = torch.device(f"cuda:{local}")
    L, d, F, B = (MODEL[n] for n in ("num_layers", "d_model", "num_features", "batch"))
    Fl = F // world
    e = ext_mod.load()
    torch.manual_seed(1 + rank)
    dec_w = [torch.empty(Fl, L - s, d, dtype=torch.bfloat16, device=dev).uniform_(-0.01, 0.01) for s in range(L)]
    Y = torch.randn(L, B, d, device=dev).bfloat16()
    bias_sum = torch.zeros(L, d, device=dev)
    sq_err = torch.zeros(L, dtype=torch.float64, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)

    class _Cfg:
        num_layers, d_model = L, d

    symm = SymmetricExchange.create(dist.group.WORLD, dev, _Cfg, B)
    sweep = []
    for density in (0.001, 0.0025, 0.005, 0.01, 0.025, 0.05):
        n = max(1, int(round(density * Fl)))                      # active features per token and layer on this rank
        cell = {"density": density, "active_per_token_per_layer_per_rank": n}
        if args.impl == "ours":
            # token-major CSR of the random selection: n features per (token, layer)
            idx = torch.rand(L, B, Fl, device=dev).topk(n, dim=-1).indices.to(torch.int32)      # [L, B, n]
            col = (idx.permute(1, 0, 2) + (torch.arange(L, device=dev, dtype=torch.int32) << 24).view(1, L, 1)).reshape(-1).contiguous()
            val = torch.rand(B * L * n, device=dev)
            tok_off = (torch.arange(B + 1, device=dev, dtype=torch.int64) * (L * n)).to(torch.int32)
            del idx

            def fused():
                e.sparse_decode(dec_w, L, B, d, Fl, 0, tok_off, col, val, None, None, None, None, None, None, None, None, None, None, 2,
                                symm.stage_ptrs, symm.rows_per_rank, rank, status)
                symm.barrier(e, status)
                e.owner_reduce_loss(symm.stage, symm.gs_ptrs, rank, bias_sum, None, Y, None, None, sq_err, symm.rows_per_rank)
                symm.barrier(e, status)

            ms = _event_ms(fused, 2, 5 if density <= 0.01 else 2)
            del col, val
        else:
            # dense activations [B, Fl] per source layer (density irrelevant for the dense kernels, kept for the table)
            acts = [torch.zeros(B, Fl, dtype=torch.bfloat16, device=dev) for _ in range(L)]
            w_t = [[dec_w[s][:, t - s, :].contiguous() for t in range(s, L)] for s in range(L)]

            def dense():
                for t in range(L):
                    out = None
                    for s in range(t + 1):
                        part = acts[s] @ w_t[s][t - s]
                        dist.all_reduce(part)                          # one all-reduce per (source, target) pair
                        out = part if out is None else out + part

            ms = _event_ms(dense, 1, 3)
            del acts, w_t
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        # bytes that have to leave one GPU: partial rows of the tokens owned elsewhere (fp32) + its share of the seed to every peer (bf16)
        nv = (world - 1) / world * L * B * d * 4 + (world - 1) * L * (B / world) * d * 2
        cell.update(ms=ms, nvlink_bytes_out_per_gpu=nv, nvlink_gbs=nv / ms / 1e6, frac_of_900_gbs=nv / ms / 1e6 / 900.0)
        sweep.append(cell)
        torch.cuda.empty_cache()
    st = int(status[0].item())
    return {"metric": f"fused sparse decode -> reduce, {L} x [{B} x {d}] outputs, ms per call (max over ranks) by density",
            "value": next(c["ms"] for c in sweep if c["density"] == 0.001), "unit": "ms", "n_gpus": world, "higher_is_better": False,
            "dtype": "bf16", "data": "synthetic (random selections, random-init weights)", "sweep": sweep, "impl": args.impl,
            "status_word": st, "config": {"model": model_name(False), "mode": "decode-reduce", "parallelism": f"tp{world}", "headline_cell": "density 0.1 %"}}


def main():
    args = parse_args()
    MODEL.clear()
    MODEL.update(SHAPES[args.shape])
    if args.batch:
        MODEL["batch"] = int(args.batch)
    MODEL["tying"] = args.decoder_tying
    MODEL["precision"] = args.precision
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return 0
    world, rank, local = setup_dist(args.gpus)
    try:
        runner = {"train": None, "inference": run_inference_sweep, "convert": run_convert, "decode-reduce": run_decode_reduce}[args.mode]
        if runner is not None:
            try:
                result = runner(args, world, rank, local)
            except Exception as exc:  # noqa: BLE001
                if args.impl != "reference":
                    raise
                result = {"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {str(exc)[:300]}"}
        elif args.impl == "reference":
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
