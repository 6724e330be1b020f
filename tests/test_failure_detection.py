"""Failure detection without faulting any GPU.

Host side (CPU, Gloo ranks as child processes): a rank that announces its departure, a rank that dies silently
between steps, and a collective that ends with an error through a short process-group timeout.
Device side: a peer barrier whose partner flag nothing ever sets runs out of its bounded wait, reports
STATUS_WAIT_TIMEOUT through the status word, and leaves the context usable.
"""
import os
import socket
import tempfile
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from crosslayer_coding_b200.parallel.health import HeartbeatMonitor, PeerLostError


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_heartbeat_detects_departure_and_lag():
    store = dist.HashStore()
    a = HeartbeatMonitor(store, 0, 2, timeout_s=0.2)
    b = HeartbeatMonitor(store, 1, 2, timeout_s=0.2)
    a.beat(0)
    b.beat(0)
    a.check(0)
    b.check(0)
    # rank 1 stops reporting: rank 0 notices after the timeout, not before
    a.beat(1)
    a.check(1)
    time.sleep(0.3)
    with pytest.raises(PeerLostError) as e:
        a.check(1)
    assert e.value.ranks == [1] and "stuck at step 0" in str(e.value)
    # an orderly departure is reported at once
    b.leave("preempted")
    with pytest.raises(PeerLostError) as e:
        a.check(3)
    assert "preempted" in str(e.value)


def _worker(rank, world, port, store_path, mode, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    hb = HeartbeatMonitor(dist.FileStore(store_path, world), rank, world, timeout_s=1.0)
    result = "finished"
    try:
        for step in range(4):
            if rank == 1 and step == 2:  # between steps, nothing in flight
                if mode == "leave":
                    hb.leave("exception in user code")
                    raise RuntimeError("simulated failure between steps")
                if mode == "die":
                    os._exit(17)  # dies silently
            hb.ready(step)  # every peer is about to launch this step too, or PeerLostError
            t = torch.ones(4) * (rank + 1)
            if mode == "collective_timeout" and rank == 1 and step == 2:
                time.sleep(6)  # never joins the collective in time
            dist.all_reduce(t)
    except PeerLostError as e:
        result = f"peer_lost:{e.ranks}"
    except RuntimeError as e:
        result = f"runtime_error:{type(e).__name__}:{str(e)[:80]}"
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(result)
    os._exit(0)  # skip the process-group teardown: the partner may be gone


@pytest.mark.parametrize("mode", ["leave", "die", "collective_timeout"])
def test_rank_failure_is_detected_on_the_host(tmp_path, mode):
    world = 2
    port = _free_port()
    store_path = os.path.join(tempfile.mkdtemp(), "hb_store")
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, store_path, mode, str(tmp_path))) for r in range(world)]
    t0 = time.time()
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung instead of reporting the failure"
    assert time.time() - t0 < 60
    r0 = open(tmp_path / "rank0.txt").read()
    if mode in ("leave", "die"):
        assert r0 == "peer_lost:[1]", r0  # noticed before step 2 was launched
    else:
        # the collective itself ends with an error after the process-group timeout
        assert r0.startswith("runtime_error"), r0


@pytest.mark.gpu
def test_bounded_peer_wait_reports_timeout_and_keeps_the_context():
    from crosslayer_coding_b200.ops import ext as ext_mod

    ext = ext_mod.load()
    dev = torch.device("cuda:0")
    # a two-rank flag table in local memory: "rank 1" does not exist, so its flag is never set
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    t0 = time.time()
    ext.peer_barrier([f.data_ptr() for f in flags], 0, 0, 1, status)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert int(status[0]) == 1, "expected STATUS_WAIT_TIMEOUT"
    assert 0.2 < waited < 10.0, waited
    # own flag was published, the partner's never arrived
    assert int(flags[0][0]) == 1 and int(flags[0][1]) == 0
    # the context is still usable
    x = torch.arange(10, device=dev).float()
    assert float((x * 2).sum()) == 90.0
    # the limit is a parameter (the staging barriers wait longer than the step's phase barriers): a quarter of the default
    status.zero_()
    t0 = time.time()
    ext.peer_barrier([f.data_ptr() for f in flags], 0, 1, 2, status, timeout_s=0.25)
    torch.cuda.synchronize()
    assert int(status[0]) == 1 and time.time() - t0 < 0.6 * max(waited, 0.5), (time.time() - t0, waited)
