"""Run a few fused BatchTopK training steps on synthetic data; the profiler range covers exactly one step.

Usage (one GPU)::

    python -m crosslayer_coding_b200.ops.profile_step --case full          # GPT-2-small shape, F=24576, k=200
    python -m crosslayer_coding_b200.ops.profile_step --case small         # same layers, F=4096, k=33
    python -m crosslayer_coding_b200.ops.profile_step --time               # CUDA-event timing per kernel group

Under Nsight Compute pass ``--profile-from-start off`` so that only the step between
``cudaProfilerStart`` and ``cudaProfilerStop`` is captured (warm-up steps run outside the range).
``--time`` prints a JSON line with CUDA-event timings (best of five after warm-up) of the encoder GEMM,
the library GEMM of the same shape, the selection stage, the decode+loss stage and the whole step.
"""
from __future__ import annotations

import argparse
import json

import torch

CASES = {
    # name: (layers, d_model, features per layer, batch tokens, k)
    "full": (12, 768, 24576, 4096, 200),
    "small": (12, 768, 4096, 4096, 33),
    "tiny": (4, 256, 2048, 1024, 16),
    "shard8": (12, 768, 3072, 4096, 25),        # one rank's share of the full case at 8 GPUs (features and k divided by 8)
    "llama-1b": (16, 2048, 32768, 4096, 200),   # Llama-3.2-1B shape: 10 G parameters, about 110 GB with fp32 moments
    "pythia-70m": (6, 512, 32768, 8192, 200),   # Pythia-70m shape with 8192-token batches (tied decoders: --tying)
    "pythia-shard8": (6, 512, 4096, 8192, 25),  # one rank's share of it at 8 GPUs
}


def build(case: str, device: torch.device, activation: str = "batchtopk", states: str = "float32", tying: str = "none",
          precision: str = "bf16", group=None):
    from .. import CLTConfig, CrossLayerTranscoder, TrainingConfig
    from ..training.fused_engine import FusedBatchTopKEngine

    L, d, F, B, k = CASES[case]
    torch.manual_seed(0)
    t16 = torch.float16 if precision == "fp16" else torch.bfloat16
    cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn=activation, batchtopk_k=k, topk_k=k,
                    clt_dtype="float16" if precision == "fp16" else "bfloat16", jumprelu_threshold=0.03, decoder_tying=tying)
    model = CrossLayerTranscoder(cfg, process_group=group, device=device)
    if tying != "none":
        with torch.no_grad():  # tied decoders start at zero
            for w in model.dec_weight:
                w.uniform_(-0.02, 0.02)
    lam = 0.0
    if activation == "jumprelu":
        # thresholds at the value that leaves about k of a token's L * F pre-activations active
        import math

        torch.manual_seed(0)
        probe = (torch.randn(512, d, device=device).to(t16) @ model.enc_weight.data[0].t()).float() + model.enc_bias.data[0].float()
        theta0 = float(torch.quantile(probe.flatten()[: 1 << 22], 1.0 - k / (L * F)))
        with torch.no_grad():
            model.log_threshold.fill_(math.log(max(theta0, 1e-6)))
        lam = 1e-3
    tc = TrainingConfig(learning_rate=1e-4, training_steps=1000, activation_path="unused", precision=precision,
                        sparsity_lambda=lam, preactivation_coef=0.0, optimizer_states_dtype=states, loss_scale_init=256.0)
    symm = None
    if group is not None:
        from ..parallel.symm import SymmetricExchange

        symm = SymmetricExchange.create(group, device, cfg, B)
    eng = FusedBatchTopKEngine(model, tc, B, symm=symm)
    torch.manual_seed(1)  # the same batch on every rank
    X = torch.randn(L, B, d, device=device).to(t16)
    Y = torch.randn(L, B, d, device=device).to(t16)
    return model, eng, X, Y


def _best_of(fn, n: int = 5) -> float:
    fn()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
    ev[0].record()
    for i in range(n):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return min(ev[i].elapsed_time(ev[i + 1]) for i in range(n))


class _TimedCalls:
    """Wraps an object so that every call of one of its functions is bracketed by a pair of CUDA events."""

    def __init__(self, inner, prefix: str, records: list):
        self._inner, self._prefix, self._records = inner, prefix, records

    def __getattr__(self, name):
        f = getattr(self._inner, name)
        if not callable(f):
            return f

        def timed(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = f(*a, **kw)
            e1.record()
            self._records.append((self._prefix + name, e0, e1))
            return r

        return timed


def tp_per_call(args) -> None:
    """CUDA-event time of every extension call, phase barrier and library collective of the tensor-parallel step, per rank
    (run under ``python -m torch.distributed.run --nproc-per-node N``; no profiler involved).  Rank 0 prints one JSON line
    with the per-call means of the slowest rank, the device time of the whole step (max over ranks) and the NVLink bytes
    that the two pushes of the decode exchange move per rank and step."""
    import collections
    import os

    import torch.distributed as dist

    from ..training import fused_engine as fe

    world, rank, local = (int(os.environ.get(n, d)) for n, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    model, eng, X, Y = build(args.case, dev, args.activation, args.optimizer_states, args.tying, args.precision, group=group)
    lam = eng.tc.sparsity_lambda
    lr = args.lr if args.lr is not None else (1e-8 if args.activation == "jumprelu" else 1e-4)
    for s in range(max(args.warmup, 3)):
        eng.train_step(X, Y, s, lr, sparsity_lambda=lam)
    torch.cuda.synchronize()
    steps = 10

    def timed_steps() -> float:
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s0.record()
        for s in range(steps):
            eng.train_step(X, Y, 100 + s, lr, sparsity_lambda=lam)
        s1.record()
        torch.cuda.synchronize()
        return s0.elapsed_time(s1) / steps

    plain_ms = timed_steps()  # without the event pairs
    records: list = []
    raw_ext = eng.ext
    eng.ext = _TimedCalls(raw_ext, "", records)
    orig_all_reduce = fe.pops.all_reduce

    def all_reduce(*a, **kw):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = orig_all_reduce(*a, **kw)
        e1.record()
        records.append(("nccl all_reduce", e0, e1))
        return r

    fe.pops.all_reduce = all_reduce
    if eng.symm is not None:
        orig_barrier = eng.symm.barrier

        def barrier(ext_obj, status):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            orig_barrier(raw_ext, status)
            e1.record()
            records.append(("peer_barrier", e0, e1))

        eng.symm.barrier = barrier
    timed_ms = timed_steps()
    eng.check_status()
    agg = collections.OrderedDict()
    for name, e0, e1 in records:
        agg.setdefault(name, [0.0, 0])
        agg[name][0] += e0.elapsed_time(e1) / steps
        agg[name][1] += 1
    names = list(agg)
    vals = torch.tensor([agg[n][0] for n in names] + [plain_ms, timed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    if rank == 0:
        L, d, F, B, k = CASES[args.case]
        push_partial = (world - 1) / world * L * B * d * 4 if world > 1 else 0       # fp32 partial sums to the owners
        push_seed = (world - 1) / world * L * B * d * 2 if world > 1 else 0          # 16-bit gradient seed to every peer
        out = {
            "case": args.case, "world": world, "activation": args.activation, "tying": args.tying, "precision": args.precision,
            "step_ms": float(vals[-2]), "step_ms_with_event_pairs": float(vals[-1]),
            "per_call_ms": {n: round(float(v), 4) for n, v in zip(names, vals[:-2].tolist())},
            "calls_per_step": {n: agg[n][1] / steps for n in names},
            "nvlink_bytes_per_rank_per_step": {"decode_partials_out": int(push_partial), "gradient_seed_out": int(push_seed)},
        }
        if world > 1:
            call = out["per_call_ms"]
            exch = call.get("sparse_decode", 0.0) + call.get("owner_reduce_loss", 0.0) + call.get("peer_barrier", 0.0)
            out["exchange_ms"] = round(exch, 4)
            out["exchange_floor_ms_at_770GBs"] = round((push_partial + push_seed) / 770e9 * 1e3, 4)
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--case", choices=sorted(CASES), default="full")
    ap.add_argument("--activation", choices=["batchtopk", "jumprelu", "topk"], default="batchtopk")
    ap.add_argument("--optimizer-states", choices=["float32", "bfloat16"], default="float32",
                    help="moment dtype of the encoder / decoder weights (bfloat16: stochastically rounded, 12 B/param/step)")
    ap.add_argument("--tying", choices=["none", "per_source", "per_target"], default="none")
    ap.add_argument("--precision", choices=["bf16", "fp16"], default="bf16")
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--dead-frac", type=float, default=0.0,
                    help="mark this fraction of every layer's features dead and train with the auxiliary loss on them")
    ap.add_argument("--preactivation-coef", type=float, default=0.0)
    ap.add_argument("--lr", type=float, default=None,
                    help="learning rate (default 1e-4; 1e-8 for jumprelu so that the active count of the synthetic data stays put)")
    ap.add_argument("--time", action="store_true", help="print CUDA-event timings instead of marking a profiler range")
    ap.add_argument("--tp-per-call", action="store_true",
                    help="per-call CUDA-event times of the tensor-parallel step (launch with torch.distributed.run, one rank per GPU)")
    args = ap.parse_args()
    if args.tp_per_call:
        tp_per_call(args)
        return
    dev = torch.device("cuda:0")
    model, eng, X, Y = build(args.case, dev, args.activation, args.optimizer_states, args.tying, args.precision)
    lam = eng.tc.sparsity_lambda
    lr = args.lr if args.lr is not None else (1e-8 if args.activation == "jumprelu" else 1e-4)
    L, d, F, B, k = CASES[args.case]
    extra = {"preactivation_coef": args.preactivation_coef}
    if args.dead_frac > 0:
        # every (1 / frac)-th feature never fires again: its encoder bias is far below the cut
        stride = max(1, int(round(1.0 / args.dead_frac)))
        with torch.no_grad():
            model.enc_bias.data[:, ::stride] = -30.0
        eng.dead_counter.view(L, -1)[:, ::stride] = 10 ** 6
        extra.update(aux_factor=1.0 / 32, dead_window=10 ** 5)
    for s in range(args.warmup):
        eng.train_step(X, Y, s, lr, sparsity_lambda=lam, **extra)
    torch.cuda.synchronize()
    if args.time:
        e = eng.ext
        step = [args.warmup]

        def full():
            eng.train_step(X, Y, step[0], lr, sparsity_lambda=lam, **extra)
            step[0] += 1

        res = {
            "case": args.case, "activation": args.activation, "optimizer_states": args.optimizer_states,
            "encoder_gemm_ms": _best_of(lambda: e.encoder_gemm(X, model.enc_weight.data, model.enc_bias.data, eng.preact, eng.status, None)),
            "library_bmm_ms": _best_of(lambda: torch.bmm(X, model.enc_weight.data.transpose(1, 2))),
            "encode_select_ms": _best_of(lambda: eng.encode_select(X)),
            "decode_loss_ms": _best_of(lambda: eng.decode_loss(Y)),
            "train_step_ms": _best_of(full, 6),
        }
        # host side of a step: enqueue time of one train_step on an idle device (nothing in it waits for the GPU)
        import time as _time

        host = []
        for _ in range(5):
            torch.cuda.synchronize()
            t0 = _time.perf_counter()
            full()
            host.append((_time.perf_counter() - t0) * 1e3)
        torch.cuda.synchronize()
        res["host_enqueue_ms"] = min(host)
        flops = 2.0 * L * B * F * d
        res["encoder_gemm_tflops"] = flops / res["encoder_gemm_ms"] / 1e9
        res["library_bmm_tflops"] = flops / res["library_bmm_ms"] / 1e9
        res["tokens_per_s"] = B / res["train_step_ms"] * 1e3
        res["active_per_token"] = int(eng.ctl[3]) / B
        eng.check_status()
        print(json.dumps(res))
        return
    torch.cuda.profiler.start()
    eng.train_step(X, Y, args.warmup, lr, sparsity_lambda=lam, **extra)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    eng.check_status()
    print(json.dumps({"case": args.case, "entries": int(eng.ctl[3]), "candidates": int(eng.ctl[4]), "fallback": int(eng.ctl[10])}))


if __name__ == "__main__":
    main()
