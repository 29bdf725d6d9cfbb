"""Process topology from the environment (reference: src/zeroband/utils/world_info.py:6-56).

torchrun provides the intra-node (local) variables; the ``GLOBAL_*`` variables describe the
DiLoCo worker this node is: one worker = one torchrun = one ZeRO-3 group."""
from __future__ import annotations

import os

_world_info: "WorldInfo | None" = None


class WorldInfo:
    world_size: int
    rank: int
    local_rank: int
    local_world_size: int

    def __init__(self):
        e = os.environ
        self.world_size = int(e["WORLD_SIZE"])
        self.rank = int(e["RANK"])
        self.local_rank = int(e["LOCAL_RANK"])
        self.local_world_size = int(e["LOCAL_WORLD_SIZE"])
        self.nnodes = self.world_size // self.local_world_size
        self.global_unique_id = e.get("GLOBAL_UNIQUE_ID", None)
        self.global_addr = e.get("GLOBAL_ADDR", None)
        self.global_port = int(e.get("GLOBAL_PORT")) if "GLOBAL_PORT" in e else None
        self.global_world_size = int(e.get("GLOBAL_WORLD_SIZE", 1))
        self.global_rank = int(e.get("GLOBAL_RANK", 0))
        # CUDA device of this process (PRIME_DEVICE_OFFSET lets several launchers share one box
        # without hiding GPUs from each other, which would break NVLink peer mappings)
        self.device_index = int(e.get("PRIME_DEVICE_OFFSET", "0")) + self.local_rank
        # Several DiLoCo workers inside ONE launcher: the job's ranks are split into
        # `workers_in_job` consecutive groups; each group is a worker (its own ZeRO-3 group) and
        # rank i of every worker forms one NVLink worker group.
        self.workers_in_job = int(e.get("PRIME_B200_WORKERS_PER_JOB", "1"))
        self.job_rank, self.job_world_size = self.rank, self.world_size
        if self.workers_in_job > 1:
            assert self.local_world_size % self.workers_in_job == 0, "workers must divide the ranks of the job evenly"
            per = self.local_world_size // self.workers_in_job
            self.global_world_size = self.workers_in_job
            self.global_rank = self.local_rank // per
            self.global_unique_id = str(self.global_rank)
            self.local_world_size = per
            self.world_size = per
            self.local_rank = self.local_rank % per
            self.rank = self.rank % per

    def __repr__(self):
        return (f"WorldInfo(world_size={self.world_size}, rank={self.rank}, local_rank={self.local_rank}, "
                f"local_world_size={self.local_world_size}, nnodes={self.nnodes}, global_unique_id={self.global_unique_id}, "
                f"global_addr={self.global_addr}, global_port={self.global_port}, global_world_size={self.global_world_size}, "
                f"global_rank={self.global_rank})")

    def json(self) -> dict[str, int | str | None]:
        return dict(self.__dict__)


def get_world_info(refresh: bool = False) -> WorldInfo:
    """Singleton; ``refresh`` re-reads the environment (tests that spawn ranks in-process use it)."""
    global _world_info
    if _world_info is None or refresh:
        _world_info = WorldInfo()
    return _world_info
