"""Per-rank logging: every record carries ``[rank r/world]``; rank 0 logs at the requested level,
the other ranks at WARNING unless ``all_ranks`` is set (so a job of eight ranks prints one copy of
its progress and every copy of its problems).  The reference prints with ``println!`` /
``eprintln!`` (plugins/model-transformer/src/lib.rs:594-597,626-630; "logging abstraction" is
unchecked in CHECKLIST.md:65)."""
from __future__ import annotations

import logging
import os
import sys
from typing import Optional

_NAME = "coeus_b200"


class _RankFilter(logging.Filter):
    def __init__(self, rank: int, world: int) -> None:
        super().__init__()
        self.rank, self.world = rank, world

    def filter(self, record: logging.LogRecord) -> bool:
        record.rank = self.rank
        record.world = self.world
        return True


def setup_logging(level: int = logging.INFO, rank: Optional[int] = None,
                  world: Optional[int] = None, all_ranks: bool = False,
                  stream=None) -> logging.Logger:
    """Configure and return the package logger (idempotent: handlers are replaced)."""
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
    log = logging.getLogger(_NAME)
    for h in list(log.handlers):
        log.removeHandler(h)
    handler = logging.StreamHandler(stream or sys.stderr)
    handler.setFormatter(logging.Formatter(
        "%(asctime)s [rank %(rank)d/%(world)d] %(levelname)s %(name)s: %(message)s"))
    handler.addFilter(_RankFilter(rank, world))
    log.addHandler(handler)
    log.setLevel(level if (rank == 0 or all_ranks) else max(level, logging.WARNING))
    log.propagate = False
    return log


def get_logger(child: Optional[str] = None) -> logging.Logger:
    return logging.getLogger(_NAME if not child else f"{_NAME}.{child}")


def log_sink(ev: dict) -> None:
    """An event-bus sink (:class:`coeus_b200.utils.metrics.EventBus`) that logs every event."""
    get_logger("events").info("%s", ev)
