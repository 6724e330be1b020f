"""Host-side failure detection for tensor-parallel jobs.

The reference has no job-level failure detection: a lost rank shows up as an NCCL timeout many minutes later
(README.md:225-231 only points at the torchrun documentation).  The fused step additionally contains kernels
that wait for peers (bounded, they give up after about a second and set a status word), so a lost rank should
be noticed on the host *before* the next step is launched.

``HeartbeatMonitor`` keeps one key per rank in the job's ``torch.distributed`` store.  Before launching step
``s`` every rank calls ``ready(s)``: it publishes ``s`` and waits until every peer has published ``s`` as well.
A peer that announced its departure with ``leave()``, or that stays behind for longer than ``timeout_s``,
makes ``ready`` raise ``PeerLostError`` naming it - with no kernel or collective of step ``s`` in flight.
Nothing here touches a GPU.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional


class PeerLostError(RuntimeError):
    def __init__(self, ranks: List[int], detail: str):
        super().__init__(f"rank(s) {ranks} lost: {detail}")
        self.ranks = ranks


class HeartbeatMonitor:
    """``store``: a ``torch.distributed`` store (``TCPStore``/``FileStore``/``HashStore``) shared by the ranks."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "clt_heartbeat"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s = float(timeout_s)
        self.prefix = prefix
        self._last_seen: Dict[int, float] = {}
        self._last_step: Dict[int, int] = {}
        self.beat(-1)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{int(step)}")

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly departure (called between steps, with nothing in flight)."""
        self.store.set(self._key(self.rank), f"gone:{reason}")

    def _read(self, r: int) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return self.store.get(self._key(r)).decode()
        except Exception:
            return None

    def check(self, step: int) -> None:
        """Raise ``PeerLostError`` if a peer left, or has not reached ``step`` within ``timeout_s`` of its last
        progress as seen from this rank."""
        now = time.monotonic()
        lost, detail = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            val = self._read(r)
            if val is None:
                first = self._last_seen.setdefault(r, now)
                if now - first > self.timeout_s:
                    lost.append(r)
                    detail.append(f"rank {r} never reported")
                continue
            if val.startswith("gone:"):
                lost.append(r)
                detail.append(f"rank {r} announced '{val[5:]}'")
                continue
            peer_step = int(val)
            if peer_step != self._last_step.get(r):
                self._last_step[r] = peer_step
                self._last_seen[r] = now
            if peer_step < step and now - self._last_seen.get(r, now) > self.timeout_s:
                lost.append(r)
                detail.append(f"rank {r} stuck at step {peer_step} (this rank is at {step})")
        if lost:
            raise PeerLostError(lost, "; ".join(detail))

    def ready(self, step: int, poll_s: float = 0.002) -> None:
        """Publish that this rank is about to launch ``step`` and block (host side) until every peer has done
        the same or is declared lost."""
        self.beat(step)
        while True:
            self.check(step)
            vals = [self._read(r) for r in range(self.world) if r != self.rank]
            if all(v is not None and not v.startswith("gone:") and int(v) >= step for v in vals):
                return
            time.sleep(poll_s)
