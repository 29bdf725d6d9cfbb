"""CUDA memory-history snapshots every `freq` steps (reference: src/zeroband/utils/profiler.py:10-60)."""
from __future__ import annotations

import os
import pickle

import torch

_MAX_ENTRIES = 10000


class MemoryProfiler:
    """Records the allocator history and dumps `<snapshot_dir>/iteration_<n>/rank<r>_memory_snapshot.pickle`
    plus a text summary each `freq` steps. On a machine without CUDA it only counts steps."""

    def __init__(self, freq: int, snapshot_dir: str, rank: int | None = None, barrier=None):
        self.freq = freq
        self.snapshot_dir = snapshot_dir
        self.step_num = 0
        self.barrier = barrier
        if rank is None:
            try:
                from .world_info import get_world_info
                rank = get_world_info().rank
            except KeyError:
                rank = 0
        self.rank = rank
        self.enabled = torch.cuda.is_available()
        if self.enabled:
            torch.cuda.memory._record_memory_history(max_entries=_MAX_ENTRIES)
        os.makedirs(snapshot_dir, exist_ok=True)

    def log_memory_summary(self, curr_snapshot_dir: str) -> None:
        summary = torch.cuda.memory_summary(device=None, abbreviated=False) if self.enabled else "no CUDA device\n"
        with open(os.path.join(curr_snapshot_dir, f"rank{self.rank}_memory_summary.txt"), "w") as f:
            f.write(summary)
        allocated = torch.cuda.memory_allocated() / 1024 ** 2 if self.enabled else 0.0
        with open(os.path.join(curr_snapshot_dir, f"rank{self.rank}_memory_allocated.txt"), "w") as f:
            f.write(f"{allocated} MB\n")

    def step(self) -> None:
        self.step_num += 1
        if self.step_num % self.freq != 0:
            return
        d = os.path.join(self.snapshot_dir, f"iteration_{self.step_num}")
        os.makedirs(d, exist_ok=True)
        if self.enabled:
            with open(os.path.join(d, f"rank{self.rank}_memory_snapshot.pickle"), "wb") as f:
                pickle.dump(torch.cuda.memory._snapshot(), f)
        self.log_memory_summary(d)
        if self.barrier is not None:
            self.barrier()
