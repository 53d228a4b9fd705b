"""The library logger: one `logging.Logger` named "primus_turbo" writing to stderr, level from PRIMUS_TURBO_LOG_LEVEL.

Call shape of the reference's logger (primus_turbo/common/logger.py): `logger.info(msg, once=..., rank=...)` and the same
for debug / warning / error / critical; `once=True` prints a given message at most once per process, `rank=r` only on
that torch.distributed rank (every rank when torch.distributed is not initialised).
"""
import logging
import os
import sys
from enum import Enum

from .constants import ENV_LOG_LEVEL


class LogLevelEnum(Enum):
    DEBUG = "DEBUG"
    INFO = "INFO"
    WARNING = "WARNING"
    ERROR = "ERROR"
    CRITICAL = "CRITICAL"

    def __str__(self) -> str:
        return self.name


class PrimusTurboLogger:
    _instance = None

    def __new__(cls, *args, **kwargs):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
        return cls._instance

    def __init__(self, name: str = "primus_turbo"):
        if getattr(self, "_ready", False):
            return
        self._ready = True
        self._seen = set()
        lg = logging.getLogger(name)
        level = getattr(logging, os.environ.get(ENV_LOG_LEVEL, "WARNING").upper(), None)
        lg.setLevel(level if isinstance(level, int) else logging.WARNING)
        lg.propagate = False
        if not lg.handlers:
            h = logging.StreamHandler(sys.stderr)
            h.setFormatter(logging.Formatter("[%(asctime)s] [%(levelname)s] [%(name)s] %(message)s", datefmt="%Y-%m-%d %H:%M:%S"))
            lg.addHandler(h)
        self._logger = lg

    @staticmethod
    def _rank() -> int:
        try:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                return dist.get_rank()
        except Exception:  # noqa: BLE001
            pass
        return 0

    def _emit(self, level: int, msg: str, once: bool, rank):
        if rank is not None and self._rank() != rank:
            return
        if once:
            key = (level, msg)
            if key in self._seen:
                return
            self._seen.add(key)
        self._logger.log(level, msg)

    def debug(self, msg, *, once=False, rank=None):
        self._emit(logging.DEBUG, msg, once, rank)

    def info(self, msg, *, once=False, rank=None):
        self._emit(logging.INFO, msg, once, rank)

    def warning(self, msg, *, once=False, rank=None):
        self._emit(logging.WARNING, msg, once, rank)

    def error(self, msg, *, once=False, rank=None):
        self._emit(logging.ERROR, msg, once, rank)

    def critical(self, msg, *, once=False, rank=None):
        self._emit(logging.CRITICAL, msg, once, rank)

    def set_level(self, level) -> None:
        self._logger.setLevel(getattr(logging, str(level).upper(), level) if not isinstance(level, int) else level)


logger = PrimusTurboLogger()
