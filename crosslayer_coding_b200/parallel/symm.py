"""Symmetric-memory exchange area for the tensor-parallel fused step.

One allocation per rank, made once, mapped into every peer (``torch.distributed._symmetric_memory``; the
kernels receive plain peer pointers).  It holds

* ``hist``   ``[rounds][world][8192]`` uint32 — histogram slots of the distributed BatchTopK threshold search,
* ``hflag``  ``[rounds][world]`` uint32 — one flag per (round, source rank) for those slots,
* ``bflag``  ``[slots][world]`` uint32 — flags of the phase barriers,
* ``stage``  ``[world][L][B/W][d]`` fp32 — partial reconstructions pushed by the peers' decode kernels,
* ``gs``     ``[L][B][d]`` bf16 — gradient seed, written by the owners of the token rows.

Every section is followed by a 256-byte guard filled with a fixed pattern; ``check_canaries`` reports the sections whose
guard was overwritten (a peer store that ran past its slot).  Compute-sanitizer cannot watch peer stores of other
processes, so this is the check that the index-checking build and the multi-GPU tests use.

Reference counterpart: the NCCL collectives C1-C4 of the reference's forward pass
(clt/models/parallel.py:143,197; clt/models/activations_local_global.py:122-123).  NCCL remains the control
plane (barriers at setup, scalar all-reduces).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

HIST_ROUNDS = 16
HIST_BINS = 8192
HIST_SLOT = HIST_BINS + 32  # a slot also carries the pool-overflow word of the selection
BARRIER_SLOTS = 4
CANARY = 0xC5  # byte pattern of the guard regions behind every section


class SymmetricExchange:
    def __init__(self, group, device: torch.device, num_layers: int, batch_tokens: int, d_model: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.L, self.B, self.d = num_layers, batch_tokens, d_model
        self.rows_per_rank = -(-batch_tokens // self.world)
        W = self.world
        # layout in bytes, every section 256-byte aligned
        def align(n: int) -> int:
            return (n + 255) // 256 * 256

        guard = 256
        self.hist_bytes = align(HIST_ROUNDS * W * HIST_SLOT * 4) + guard
        self.hflag_bytes = align(HIST_ROUNDS * W * 4) + guard
        self.bflag_bytes = align(BARRIER_SLOTS * W * 4) + guard
        self.stage_bytes = align(W * num_layers * self.rows_per_rank * d_model * 4) + guard
        self.gs_bytes = align(num_layers * batch_tokens * d_model * 2) + guard
        total = self.hist_bytes + self.hflag_bytes + self.bflag_bytes + self.stage_bytes + self.gs_bytes
        self.buffer = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group)
        base: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        o_hflag = self.hist_bytes
        o_bflag = o_hflag + self.hflag_bytes
        o_stage = o_bflag + self.bflag_bytes
        o_gs = o_stage + self.stage_bytes
        self.hist_data_ptrs = base
        self.hist_flag_ptrs = [b + o_hflag for b in base]
        self.barrier_flag_ptrs = [b + o_bflag for b in base]
        self.stage_ptrs = [b + o_stage for b in base]
        self.gs_ptrs = [b + o_gs for b in base]
        self.slot_elems = HIST_SLOT
        self.stage = self.buffer[o_stage : o_stage + W * num_layers * self.rows_per_rank * d_model * 4].view(torch.float32)
        self.gs = self.buffer[o_gs : o_gs + num_layers * batch_tokens * d_model * 2].view(torch.bfloat16).view(num_layers, batch_tokens, d_model)
        self._guards = {}
        end = 0
        for name, nbytes in (("hist", self.hist_bytes), ("hflag", self.hflag_bytes), ("bflag", self.bflag_bytes), ("stage", self.stage_bytes),
                             ("gs", self.gs_bytes)):
            end += nbytes
            self._guards[name] = self.buffer[end - guard: end]
            self._guards[name].fill_(CANARY)
        self.barrier_seq = 0
        self.supports_reduce = True
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank has zeroed its flags before anyone signals

    @classmethod
    def create(cls, group, device, clt_config, batch_tokens: int) -> "SymmetricExchange":
        return cls(group, torch.device(device), clt_config.num_layers, batch_tokens, clt_config.d_model)

    def check_canaries(self):
        """Names of the sections whose guard bytes no longer hold the pattern (host read; for tests and debug runs)."""
        return [name for name, g in self._guards.items() if not bool((g == CANARY).all().item())]

    def barrier(self, ext, status: torch.Tensor) -> None:
        """Cross-GPU phase barrier on the current stream (one tiny kernel, bounded wait)."""
        self.barrier_seq += 1
        ext.peer_barrier(self.barrier_flag_ptrs, self.rank, self.barrier_seq % BARRIER_SLOTS, self.barrier_seq, status)
