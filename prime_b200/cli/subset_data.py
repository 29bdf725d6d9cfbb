"""List (and optionally fetch) the parquet shards one data rank would read: files
``data_rank :: data_world_size`` of each dataset (reference: scripts/subset_data.py:79-107).

    python -m prime_b200.cli.subset_data --dataset /data/fineweb-edu --data-rank 1 --data-world-size 8 [--copy-to /local/subset]
"""
from __future__ import annotations

import argparse
import os
import shutil

from ..data import _get_datafiles


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True, help="comma-separated dataset paths / names")
    ap.add_argument("--data-rank", type=int, required=True)
    ap.add_argument("--data-world-size", type=int, required=True)
    ap.add_argument("--max-shards", type=int, default=None)
    ap.add_argument("--copy-to", default=None)
    a = ap.parse_args()
    for ds in a.dataset.split(","):
        files = _get_datafiles(ds)[a.data_rank::a.data_world_size]
        if a.max_shards is not None:
            files = files[: a.max_shards]
        for f in files:
            print(f)
            if a.copy_to and os.path.exists(f):
                dst = os.path.join(a.copy_to, os.path.basename(ds.rstrip("/")), os.path.basename(f))
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                shutil.copy2(f, dst)


if __name__ == "__main__":
    main()
