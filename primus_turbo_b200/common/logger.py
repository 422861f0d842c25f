"""Library logger: level from ``PRIMUS_TURBO_LOG_LEVEL`` (default WARNING), messages to stderr, and the
two per-call filters of the reference's logger (primus_turbo/common/logger.py:29-130): ``once=True``
emits a (level, message) pair at most once per process, ``rank=r`` only on distributed rank ``r``."""

from __future__ import annotations

import logging
import os
import sys

ENV_LOG_LEVEL = "PRIMUS_TURBO_LOG_LEVEL"  # primus_turbo/common/constants.py:16


class _Logger:
    def __init__(self, name: str = "primus_turbo"):
        level = getattr(logging, os.environ.get(ENV_LOG_LEVEL, "WARNING").upper(), None)
        self._log = logging.getLogger(name)
        self._log.setLevel(level if isinstance(level, int) else logging.WARNING)
        self._log.propagate = False
        if not self._log.handlers:
            h = logging.StreamHandler(sys.stderr)
            h.setFormatter(logging.Formatter("[%(asctime)s][%(name)s][%(levelname)s] %(message)s", datefmt="%H:%M:%S"))
            self._log.addHandler(h)
        self._seen = set()

    @staticmethod
    def _rank() -> int:
        try:
            import torch.distributed as dist

            return dist.get_rank() if dist.is_initialized() else 0
        except Exception:  # noqa: BLE001
            return 0

    def set_level(self, level: int) -> None:
        self._log.setLevel(level)

    def log(self, level: int, msg: str, *args, once: bool = False, rank=None, **kwargs) -> None:
        if rank is not None and self._rank() != rank:
            return
        if once:
            if (level, msg) in self._seen:
                return
            self._seen.add((level, msg))
        self._log.log(level, msg, *args, **kwargs)

    def debug(self, msg, *a, once=False, rank=None, **k):
        self.log(logging.DEBUG, msg, *a, once=once, rank=rank, **k)

    def info(self, msg, *a, once=False, rank=None, **k):
        self.log(logging.INFO, msg, *a, once=once, rank=rank, **k)

    def warning(self, msg, *a, once=False, rank=None, **k):
        self.log(logging.WARNING, msg, *a, once=once, rank=rank, **k)

    def error(self, msg, *a, once=False, rank=None, **k):
        self.log(logging.ERROR, msg, *a, once=once, rank=rank, **k)


logger = _Logger()
