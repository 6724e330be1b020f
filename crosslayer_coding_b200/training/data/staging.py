"""Pinned host ring + side-stream host->device copies for activation batches.

The reference store moves every (layer, chunk) slice with a synchronous pageable ``.to(device)``
(clt/training/data/manifest_activation_store.py:894-895).  Here a batch is assembled in one pinned
buffer ``[2, L, B, d]`` (inputs, targets), copied with a single ``cudaMemcpyAsync`` on a dedicated
stream into one of ``depth`` device slots, and handed to the training stream through an event, so the
copy of batch ``i+1`` overlaps the step on batch ``i``.  On CPU the stager degenerates to a no-op.

Sharded staging (tensor-parallel jobs): every rank needs the whole batch, but all ranks of a node pull it
from the same host memory, and W full copies over PCIe cost W times the bytes of one.  With ``shard_group``
each rank copies only its ``1/W`` slice of the token rows host->device and the slices are all-gathered over
NVLink on the staging stream (a communicator of its own, so the gather never interleaves with the training
step's collectives), followed by one device-side re-layout into ``[..., B, d]``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch


class DeviceStager:
    def __init__(self, shape: Tuple[int, ...], dtype: torch.dtype, device: torch.device, depth: int = 3,
                 shard_group=None, row_dim: int = 2):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.depth = max(2, depth)
        self.shape = tuple(shape)
        self.dtype = dtype
        self.bytes_per_batch = int(torch.tensor([], dtype=dtype).element_size()) * int(torch.Size(shape).numel())
        if self.cuda:
            self.host = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(self.depth)]
            self.dev = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(self.depth)]
            # high priority: the copy / gather kernels are tiny and should slip in between the step's long kernels
            self.stream = torch.cuda.Stream(device=self.device, priority=-1)
            self.copied: List[Optional[torch.cuda.Event]] = [None] * self.depth
            self.released: List[Optional[torch.cuda.Event]] = [None] * self.depth
            self._init_shard(shard_group, row_dim)
        else:
            # CPU: the "device" slot is the host buffer itself; several slots so a producer thread never
            # overwrites a batch the consumer still holds
            self.host = [torch.empty(shape, dtype=dtype) for _ in range(self.depth)]
            self.dev = list(self.host)
        self._next = 0
        if not self.cuda:
            self.shard_world = 1

    def _init_shard(self, shard_group, row_dim: int) -> None:
        """Collective over ``shard_group``: creates the staging communicator and the gather buffers."""
        import torch.distributed as dist

        self.shard_world, self.shard_rank, self.gather_group = 1, 0, None
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
        self.piece = [torch.empty(self.outer, self.rows_per_rank, self.inner, dtype=self.dtype, device=self.device) for _ in range(self.depth)]
        self.gathered = torch.empty(W, self.outer, self.rows_per_rank, self.inner, dtype=self.dtype, device=self.device)

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
            host = self.host[slot] if src is None else src
            if self.shard_world == 1:
                self.dev[slot].copy_(host, non_blocking=True)
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
        return self.dev[slot]

    def release(self, slot: int) -> None:
        """Mark the device slot reusable once the work queued so far on the current stream is done."""
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.released[slot] = ev
