"""Fast-forward the dataloader N steps and write ``data/_{rank}.pt`` files, so a run can resume with a
different data position (reference: scripts/skip_data.py:31-76).

    python -m prime_b200.cli.skip_data @cfg.toml --steps 1000 --out /data/skip_ckpt [--ranks 8]
"""
from __future__ import annotations

import os

import torch

from ..checkpoint import CkptManager
from ..config import Config, parse_argv
from ..data import get_dataloader
from ..train import _get_tokenizer


class SkipConfig(Config):
    steps: int
    out: str
    ranks: int = 1


def skip(config: SkipConfig) -> list[str]:
    tokenizer = _get_tokenizer(config)
    written = []
    batch = config.optim.batch_size // config.ranks
    for rank in range(config.ranks):
        dl = get_dataloader(tokenizer, world_size=config.ranks, rank=rank, batch_size=batch, data_config=config.data, device="cpu")
        it = iter(dl)
        for _ in range(config.steps):
            next(it)
        d = os.path.join(config.out, "data")
        CkptManager.save_data(d, dl, rank)
        written.append(os.path.join(d, f"_{rank}.pt"))
    return written


def main(argv=None):
    cfg = SkipConfig(**parse_argv(argv))
    for p in skip(cfg):
        print(p)


if __name__ == "__main__":
    main()
