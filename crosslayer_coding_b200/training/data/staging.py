"""Pinned host ring + side-stream host->device copies for activation batches.

The reference store moves every (layer, chunk) slice with a synchronous pageable ``.to(device)``
(clt/training/data/manifest_activation_store.py:894-895).  Here a batch is assembled in one pinned
buffer ``[2, L, B, d]`` (inputs, targets), copied with a single ``cudaMemcpyAsync`` on a dedicated
stream into one of ``depth`` device slots, and handed to the training stream through an event, so the
copy of batch ``i+1`` overlaps the step on batch ``i``.  On CPU the stager degenerates to a no-op.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch


class DeviceStager:
    def __init__(self, shape: Tuple[int, ...], dtype: torch.dtype, device: torch.device, depth: int = 3):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.depth = max(2, depth)
        self.shape = tuple(shape)
        self.dtype = dtype
        self.bytes_per_batch = int(torch.tensor([], dtype=dtype).element_size()) * int(torch.Size(shape).numel())
        if self.cuda:
            self.host = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(self.depth)]
            self.dev = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(self.depth)]
            self.stream = torch.cuda.Stream(device=self.device)
            self.copied: List[Optional[torch.cuda.Event]] = [None] * self.depth
            self.released: List[Optional[torch.cuda.Event]] = [None] * self.depth
        else:
            # CPU: the "device" slot is the host buffer itself; several slots so a producer thread never
            # overwrites a batch the consumer still holds
            self.host = [torch.empty(shape, dtype=dtype) for _ in range(self.depth)]
            self.dev = list(self.host)
        self._next = 0

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
            self.dev[slot].copy_(self.host[slot] if src is None else src, non_blocking=True)
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
