"""Deterministic (chunk, row) batch sampler for manifest datasets.

Behaviour follows the reference ``ChunkRowSampler`` (clt/training/data/manifest_activation_store.py:41-322):
yields ``(batch, 2)`` uint32 arrays ``[chunk_id, row_id]``; ``sequential`` walks the chunks in a random
order and takes contiguous full batches from each chunk's shuffled rows (the tail of a chunk is dropped);
``random_chunk`` draws every batch from a random chunk that still has a full batch left; with
``shard_data`` each rank owns rows ``rank::world`` of every chunk.

Design difference: a chunk's row permutation is a pure function of ``(seed, epoch, chunk_id)``, so the
checkpointed state is a handful of counters instead of every permutation (the reference serialises all
per-chunk permutations, i.e. one integer per token of the dataset).
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, Optional, Union

import numpy as np


class ChunkRowSampler:
    def __init__(
        self,
        chunk_sizes: Union[Dict[int, int], np.ndarray],
        num_chunks: int,
        batch: int,
        seed: int,
        epoch: int,
        rank: int,
        world: int,
        sampling_strategy: str = "sequential",
        shard_data: bool = True,
        initial_sampler_state: Optional[Dict[str, Any]] = None,
    ):
        if isinstance(chunk_sizes, dict):
            sizes = {int(k): int(v) for k, v in chunk_sizes.items()}
        else:
            sizes = {i: int(s) for i, s in enumerate(chunk_sizes) if s > 0}
        self.chunk_sizes = {c: n for c, n in sizes.items() if c < num_chunks}
        if not self.chunk_sizes:
            raise ValueError("chunk_sizes cannot be empty")
        if batch <= 0:
            raise ValueError("batch size must be positive")
        if not 0 <= rank < world:
            raise ValueError(f"Invalid rank/world: {rank}/{world}")
        if sampling_strategy not in ("sequential", "random_chunk"):
            raise ValueError(f"Invalid sampling_strategy: '{sampling_strategy}'. Must be 'sequential' or 'random_chunk'.")
        self.num_chunks = num_chunks
        self.batch = int(batch)
        self.seed = int(seed)
        self.epoch = int(epoch)
        self.rank = rank
        self.world = world
        self.sampling_strategy = sampling_strategy
        self.shard_data = shard_data
        self._perm_cache: Dict[int, np.ndarray] = {}
        self._begin_epoch()
        if initial_sampler_state:
            self.load_state_dict(initial_sampler_state)

    # ------------------------------------------------------------------ epoch state
    def _rows_owned(self, chunk_id: int) -> int:
        n = self.chunk_sizes[chunk_id]
        if not self.shard_data:
            return n
        return len(range(self.rank, n, self.world))

    def _chunk_rows(self, chunk_id: int) -> np.ndarray:
        rows = self._perm_cache.get(chunk_id)
        if rows is None:
            n = self.chunk_sizes[chunk_id]
            base = np.arange(n, dtype=np.uint32)
            if self.shard_data:
                base = base[self.rank :: self.world]
            rng = np.random.default_rng([self.seed, self.epoch, chunk_id, 0x5EED])
            rows = rng.permutation(base).astype(np.uint32)
            if len(self._perm_cache) > 8:  # a few chunks are live at a time
                self._perm_cache.pop(next(iter(self._perm_cache)))
            self._perm_cache[chunk_id] = rows
        return rows

    def _begin_epoch(self) -> None:
        self._perm_cache.clear()
        self.rng = np.random.default_rng([self.seed, self.epoch])
        owned = {c: self._rows_owned(c) for c in sorted(self.chunk_sizes)}
        self._owned = owned
        self.total_rows_this_rank = sum(owned.values())
        self.total_batches_this_rank = sum(n // self.batch for n in owned.values())
        usable = [c for c, n in owned.items() if n > 0]
        self.chunk_order = self.rng.permutation(np.array(usable, dtype=np.int64)) if usable else np.zeros(0, dtype=np.int64)
        self.cursor_chunk = 0          # sequential: index into chunk_order
        self.cursor_row = 0            # sequential: offset inside the current chunk
        self.offsets = {c: 0 for c in owned}  # random_chunk: rows consumed per chunk
        self.batches_yielded = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)
        self._begin_epoch()

    # -------------------------------------------------------------------- iteration
    def __iter__(self) -> Iterator[np.ndarray]:
        return self

    def __len__(self) -> int:
        return self.total_batches_this_rank

    def _emit(self, chunk_id: int, start: int) -> np.ndarray:
        rows = self._chunk_rows(chunk_id)[start : start + self.batch]
        out = np.empty((self.batch, 2), dtype=np.uint32)
        out[:, 0] = chunk_id
        out[:, 1] = rows
        self.batches_yielded += 1
        return out

    def __next__(self) -> np.ndarray:
        if self.sampling_strategy == "sequential":
            while self.cursor_chunk < len(self.chunk_order):
                cid = int(self.chunk_order[self.cursor_chunk])
                if self.cursor_row + self.batch <= self._owned[cid]:
                    start = self.cursor_row
                    self.cursor_row += self.batch
                    if self.cursor_row >= self._owned[cid]:
                        self.cursor_chunk += 1
                        self.cursor_row = 0
                    return self._emit(cid, start)
                self.cursor_chunk += 1
                self.cursor_row = 0
            raise StopIteration
        # random_chunk
        avail = [c for c, n in self._owned.items() if self.offsets[c] + self.batch <= n]
        if not avail or self.batches_yielded >= self.total_batches_this_rank:
            raise StopIteration
        cid = int(self.rng.choice(avail))
        start = self.offsets[cid]
        self.offsets[cid] = start + self.batch
        return self._emit(cid, start)

    # ------------------------------------------------------------------------ state
    def state_dict(self) -> Dict[str, Any]:
        return {
            "epoch": self.epoch,
            "seed": self.seed,
            "sampling_strategy": self.sampling_strategy,
            "shard_data": self.shard_data,
            "rank": self.rank,
            "world": self.world,
            "batch": self.batch,
            "rng_state": self.rng.bit_generator.state,
            "chunk_order": self.chunk_order.tolist(),
            "cursor_chunk": self.cursor_chunk,
            "cursor_row": self.cursor_row,
            "offsets": {int(k): int(v) for k, v in self.offsets.items()},
            "batches_yielded": self.batches_yielded,
        }

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self.seed = int(state.get("seed", self.seed))
        self.sampling_strategy = state.get("sampling_strategy", self.sampling_strategy)
        self.set_epoch(int(state["epoch"]))
        self.rng.bit_generator.state = state["rng_state"]
        self.chunk_order = np.array(state["chunk_order"], dtype=np.int64)
        self.cursor_chunk = int(state["cursor_chunk"])
        self.cursor_row = int(state["cursor_row"])
        self.offsets = {int(k): int(v) for k, v in state["offsets"].items()}
        self.batches_yielded = int(state["batches_yielded"])
