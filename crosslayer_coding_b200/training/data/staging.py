"""Pinned host ring + side-stream host->device copies for activation batches.

The reference store moves every (layer, chunk) slice with a synchronous pageable ``.to(device)``
(clt/training/data/manifest_activation_store.py:894-895).  Here a batch is assembled in one pinned
buffer ``[2, L, B, d]`` (inputs, targets), copied with a single ``cudaMemcpyAsync`` on a dedicated
stream into one of ``depth`` device slots, and handed to the training stream through an event, so the
copy of batch ``i+1`` overlaps the step on batch ``i``.  On CPU the stager degenerates to a no-op.

Sharded staging (tensor-parallel jobs): every rank needs the whole batch, but all ranks of a node pull it
from the same host memory, and W full copies over PCIe cost W times the bytes of one.  With ``shard_group``
each rank copies only its ``1/W`` slice of the token rows host->device and the slices travel to the peers over
NVLink on the staging stream:

* **push** (default): the device slots live in symmetric memory; a rank copies its rows from the pinned buffer
  straight into their final place in its own slot (one strided copy) and then into the same place of every
  peer's slot (one strided peer copy each).  All of it runs on the copy engines: no SM is taken from the
  training step and no re-layout pass is needed.  Two flag barriers (one-warp kernels on the staging stream
  with flags of their own in the same symmetric allocation; they need no shared memory, so they start beside
  the step's persistent kernels) bracket the copies: "every rank has released this slot" before, "every push
  has landed" after.  Their waits are bounded (``barrier_timeout_s``, long enough for a peer's slow data
  loader); a wait that runs out sets the stager's status word, which ``check_status`` turns into an error.
* **gather** (fallback when symmetric memory cannot be set up): NCCL all-gather of the slices followed by one
  device-side re-layout into ``[..., B, d]``.
"""
from __future__ import annotations

import logging
from typing import List, Optional, Tuple

import torch

logger = logging.getLogger(__name__)


class DeviceStager:
    def __init__(self, shape: Tuple[int, ...], dtype: torch.dtype, device: torch.device, depth: int = 3,
                 shard_group=None, row_dim: int = 2, barrier_timeout_s: float = 60.0):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.depth = max(2, depth)
        self.barrier_timeout_s = float(barrier_timeout_s)
        self._acquired = 0
        self.shape = tuple(shape)
        self.dtype = dtype
        self.bytes_per_batch = int(torch.tensor([], dtype=dtype).element_size()) * int(torch.Size(shape).numel())
        if self.cuda:
            self.host = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(self.depth)]
            self.dev: List[torch.Tensor] = []
            self.push = False
            # high priority: the copy / gather kernels are tiny and should slip in between the step's long kernels
            self.stream = torch.cuda.Stream(device=self.device, priority=-1)
            self.copied: List[Optional[torch.cuda.Event]] = [None] * self.depth
            self.released: List[Optional[torch.cuda.Event]] = [None] * self.depth
            self._init_shard(shard_group, row_dim)
            if not self.dev:
                self.dev = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(self.depth)]
        else:
            # CPU: the "device" slot is the host buffer itself; several slots so a producer thread never
            # overwrites a batch the consumer still holds
            self.host = [torch.empty(shape, dtype=dtype) for _ in range(self.depth)]
            self.dev = list(self.host)
        self._next = 0
        # optional callable returning the CUDA event a copy has to wait for before it starts (the consumer can place the
        # copies in a phase of its step where the extra memory traffic costs least)
        self.gate = None
        if not self.cuda:
            self.shard_world = 1

    def _init_shard(self, shard_group, row_dim: int) -> None:
        """Collective over ``shard_group``: creates the staging communicator and the gather buffers."""
        import torch.distributed as dist

        self.shard_world, self.shard_rank, self.gather_group = 1, 0, None
        self.peer_outer: Optional[int] = None  # leading outer indices whose rows the peers receive (None: all of them)
        if shard_group is None or not dist.is_initialized() or dist.get_world_size(shard_group) <= 1:
            return
        W = dist.get_world_size(shard_group)
        rows = self.shape[row_dim]
        if rows % W != 0:
            return
        self.shard_world, self.shard_rank = W, dist.get_rank(shard_group)
        self.gather_group = dist.new_group(ranks=dist.get_process_group_ranks(shard_group), backend="nccl")
        self.row_dim = row_dim
        self.outer = int(torch.Size(self.shape[:row_dim]).numel())
        self.inner = int(torch.Size(self.shape[row_dim + 1:]).numel())
        self.rows, self.rows_per_rank = rows, rows // W
        self.push = self._init_push(shard_group)
        if self.push:
            return
        self.piece = [torch.empty(self.outer, self.rows_per_rank, self.inner, dtype=self.dtype, device=self.device) for _ in range(self.depth)]
        self.gathered = torch.empty(W, self.outer, self.rows_per_rank, self.inner, dtype=self.dtype, device=self.device)

    def _init_push(self, shard_group) -> bool:
        """Device slots in symmetric memory, mapped into every peer of ``shard_group``.  Collective."""
        import torch.distributed as dist

        ok = 1
        try:
            import torch.distributed._symmetric_memory as symm_mem

            from ...ops import ext as ext_mod

            self._ext = ext_mod.load()
            slot_bytes = (self.bytes_per_batch + 255) // 256 * 256
            flag_bytes = 4096  # [4 slots][world] uint32 barrier flags behind the batch slots
            buf = symm_mem.empty(self.depth * slot_bytes + flag_bytes, dtype=torch.uint8, device=self.device)
            buf[self.depth * slot_bytes:].zero_()
            torch.cuda.synchronize(self.device)
            handle = symm_mem.rendezvous(buf, shard_group)
            self._symm_buf, self._symm_handle, self._slot_bytes = buf, handle, slot_bytes
            self._peer_base = [int(p) for p in handle.buffer_ptrs]
            self._flag_ptrs = [b + self.depth * slot_bytes for b in self._peer_base]
            self._barrier_seq = 0
            self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
            self.dev = [buf[i * slot_bytes: i * slot_bytes + self.bytes_per_batch].view(self.dtype).view(self.shape) for i in range(self.depth)]
        except Exception as e:  # no symmetric memory on this system: NCCL all-gather instead
            logger.warning("sharded staging falls back to the NCCL all-gather (%s: %s)", type(e).__name__, e)
            ok = 0
        # the same path on every rank; the all-reduce also orders "flags zeroed" before anybody's first signal
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.gather_group)
        if int(flag.item()) == 0:
            self.dev = []
            return False
        return True

    def push_only_leading(self, outer_count: Optional[int]) -> bool:
        """Restrict the peer pushes to the first ``outer_count`` outer indices; the remaining ones (the target half of an
        ``[2, L, B, d]`` batch when ``outer_count == L``) stay valid on the rank that loaded the rows only.  For consumers
        that need every token's inputs but only their own token rows of the targets (the tensor-parallel fused step: the
        loss of a token is finished by the rank that owns its row block, the same block this stager loads).  Returns
        whether the restriction is in force (push staging only)."""
        if not (self.cuda and getattr(self, "push", False)):
            return False
        self.peer_outer = None if outer_count is None else max(0, min(int(outer_count), self.outer))
        return self.peer_outer is not None

    def _push_rows(self, slot: int, host: torch.Tensor) -> None:
        """Own rows: pinned host -> own slot -> every peer's slot, as strided copies on the staging stream."""
        es = host.element_size()
        width = self.rows_per_rank * self.inner * es          # bytes of this rank's rows per outer index
        pitch = self.rows * self.inner * es
        off = self.shard_rank * width
        mine = self.dev[slot].data_ptr() + off
        self._barrier()                                        # every rank's consumer has released this slot
        self._ext.memcpy_2d(mine, pitch, host.data_ptr() + off, pitch, width, self.outer)
        height = self.outer if self.peer_outer is None else self.peer_outer
        for i in range(1, self.shard_world):
            if height == 0:
                break
            p = (self.shard_rank + i) % self.shard_world       # staggered: no two ranks start on the same peer
            self._ext.memcpy_2d(self._peer_base[p] + slot * self._slot_bytes + off, pitch, mine, pitch, width, height)
        self._barrier()                                        # every rank's pushes have landed

    def _barrier(self) -> None:
        self._barrier_seq += 1
        self._ext.peer_barrier(self._flag_ptrs, self.shard_rank, self._barrier_seq % 4, self._barrier_seq, self.status,
                               self.barrier_timeout_s)

    def check_status(self) -> None:
        """Host read (synchronising) of the staging barriers' status word."""
        if self.cuda and getattr(self, "push", False):
            code = int(self.status[0].item())
            if code != 0:
                self.status.zero_()
                raise RuntimeError(f"staging barrier of rank {self.shard_rank} ran out of its {self.barrier_timeout_s:.0f} s wait "
                                   "(a peer stopped submitting batches)")

    @property
    def h2d_bytes_per_rank(self) -> int:
        return self.bytes_per_batch // max(1, getattr(self, "shard_world", 1))

    def host_slot(self) -> Tuple[int, torch.Tensor]:
        """Pinned buffer to fill for the next batch.  Blocks (host side) only until the copy that last
        used this slot has left the host buffer."""
        i = self._next
        self._next = (self._next + 1) % self.depth
        if self.cuda and self.copied[i] is not None:
            self.copied[i].synchronize()
        return i, self.host[i]

    def submit(self, slot: int, src: Optional[torch.Tensor] = None) -> None:
        """Start the async copy of host slot ``slot`` (or of the pinned tensor ``src``) to its device slot."""
        if not self.cuda:
            if src is not None:
                self.dev[slot] = src
            return
        with torch.cuda.stream(self.stream):
            if self.released[slot] is not None:
                self.stream.wait_event(self.released[slot])  # consumer is done with the old contents
            gate = self.gate() if self.gate is not None else None
            if gate is not None:
                self.stream.wait_event(gate)
            host = self.host[slot] if src is None else src
            if self.shard_world == 1:
                self.dev[slot].copy_(host, non_blocking=True)
            elif self.push:
                assert host.is_contiguous() and tuple(host.shape) == self.shape and host.dtype == self.dtype
                self._push_rows(slot, host)
            else:
                import torch.distributed as dist

                # this rank's rows only: one contiguous copy per outer index (a strided pinned source would be
                # made contiguous on the host first)
                r0 = self.shard_rank * self.rows_per_rank
                hv = host.view(self.outer, self.rows, self.inner)
                for o in range(self.outer):
                    self.piece[slot][o].copy_(hv[o, r0:r0 + self.rows_per_rank], non_blocking=True)
                dist.all_gather_into_tensor(self.gathered, self.piece[slot], group=self.gather_group)
                self.dev[slot].view(self.outer, self.shard_world, self.rows_per_rank, self.inner).copy_(self.gathered.permute(1, 0, 2, 3))
            ev = torch.cuda.Event()
            ev.record(self.stream)
            self.copied[slot] = ev

    def acquire(self, slot: int) -> torch.Tensor:
        """Device tensor of ``slot``; the current stream waits for its copy."""
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_event(self.copied[slot])
            self._acquired += 1
            if self._acquired % 512 == 0:
                self.check_status()
        return self.dev[slot]

    def release(self, slot: int) -> None:
        """Mark the device slot reusable once the work queued so far on the current stream is done."""
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.released[slot] = ev
