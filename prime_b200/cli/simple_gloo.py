"""Smallest possible connectivity check between two hosts: a TCPStore on ``MASTER_ADDR`` and a gloo process
group built on it by hand, the way the elastic mesh builds its global group (reference: scripts/simple_gloo.py:10-17).

    MASTER_ADDR=10.0.0.1 RANK=0 WORLD_SIZE=2 python -m prime_b200.cli.simple_gloo      # and RANK=1 on the peer
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def main() -> float:
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "12345"))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore(host_name=addr, port=port, is_master=(rank == 0), world_size=world,
                          timeout=datetime.timedelta(seconds=60))
    store.set(f"hello_{rank}", "1")
    pg = dist.ProcessGroupGloo(dist.PrefixStore("simple_gloo", store), rank, world, datetime.timedelta(seconds=60))
    t = torch.ones(4) * (rank + 1)
    pg.allreduce([t]).wait()
    print(f"[rank {rank}] store ok, gloo all-reduce ok: {t.tolist()}")
    del pg
    return float(t[0])


if __name__ == "__main__":
    main()
