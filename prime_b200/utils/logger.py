"""Rank-aware logging (reference: src/zeroband/utils/logger.py:15-55): `[Rank n]` prefix, non-zero
local ranks silenced unless `log_all_rank`."""
from __future__ import annotations

import logging
import os

_logger: logging.Logger | None = None


class _RankFormatter(logging.Formatter):
    def __init__(self, local_rank: int):
        super().__init__()
        self.local_rank = local_rank

    def format(self, record):
        fmt = "{asctime} [{levelname}] [Rank " + str(self.local_rank) + "] {message}"
        return logging.Formatter(fmt, style="{", datefmt="%H:%M:%S").format(record)


def get_logger(config=None, name: str | None = None) -> logging.Logger:
    global _logger
    if _logger is not None:
        return _logger
    try:
        from .world_info import get_world_info
        local_rank = get_world_info().local_rank
    except KeyError:
        local_rank = 0
    logger = logging.getLogger(name or __name__)
    log_level = config.log_level if config is not None else os.environ.get("ZERO_BAND_LOG_LEVEL", "INFO")
    log_all = config.log_all_rank if config is not None else os.environ.get("ZERO_BAND_LOG_ALL_RANK", "false").lower() in ("1", "true")
    if local_rank == 0 or log_all:
        logger.setLevel(getattr(logging, log_level, logging.INFO))
    else:
        logger.setLevel(logging.CRITICAL)
    handler = logging.StreamHandler()
    handler.setFormatter(_RankFormatter(local_rank))
    logger.addHandler(handler)
    logger.propagate = False
    _logger = logger
    return logger


def reset_logger() -> None:
    global _logger
    if _logger is not None:
        for h in list(_logger.handlers):
            _logger.removeHandler(h)
    _logger = None
