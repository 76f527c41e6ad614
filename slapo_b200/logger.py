"""Rank-aware logging.

``get_logger(name)`` hands out one logger per name.  Every logging method
takes two extra keyword arguments: ``ranks`` (an int or a list of ints, the
ranks that may print; default all) and ``group`` (the process group the ranks
are counted in).  When torch.distributed is initialised every record is
prefixed with ``[Rank n]``.

Parity: slapo/logger.py:30-79 of the reference.
"""
from __future__ import annotations

import logging
import sys

_LOGGERS: dict[str, "RankLogger"] = {}


def _dist_rank(group=None):
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(group)
    except Exception:  # pragma: no cover - torch missing or group invalid
        pass
    return None


class RankLogger(logging.LoggerAdapter):
    """A ``logging.Logger`` front that filters records by rank."""

    def __init__(self, name, level):
        base = logging.getLogger(f"slapo_b200.{name}")
        base.setLevel(level)
        base.propagate = False
        if not base.handlers:
            handler = logging.StreamHandler(sys.stderr)
            handler.setFormatter(
                logging.Formatter(
                    "[%(asctime)s] %(levelname)s %(name)s: %(message)s", "%H:%M:%S"
                )
            )
            base.addHandler(handler)
        super().__init__(base, {})

    def log(self, level, msg, *args, ranks=None, group=None, **kwargs):
        rank = _dist_rank(group)
        if ranks is not None and rank is not None:
            allowed = [ranks] if isinstance(ranks, int) else list(ranks)
            if rank not in allowed:
                return
        if rank is not None:
            msg = f"[Rank {rank}] {msg}"
        if self.isEnabledFor(level):
            self.logger.log(level, msg, *args, **kwargs)

    def debug(self, msg, *args, **kwargs):
        self.log(logging.DEBUG, msg, *args, **kwargs)

    def info(self, msg, *args, **kwargs):
        self.log(logging.INFO, msg, *args, **kwargs)

    def warning(self, msg, *args, **kwargs):
        self.log(logging.WARNING, msg, *args, **kwargs)

    def error(self, msg, *args, **kwargs):
        self.log(logging.ERROR, msg, *args, **kwargs)


def get_logger(name: str = "Slapo", level=logging.INFO) -> RankLogger:
    if name not in _LOGGERS:
        _LOGGERS[name] = RankLogger(name, level)
    return _LOGGERS[name]
