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
