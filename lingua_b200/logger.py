"""Logging set-up for multi-rank jobs: every record is prefixed with rank, level, wall time and
time since start; continuation lines are indented under the prefix; stdout gets everything,
stderr warnings and above, and rank 0 also appends to a file (lingua/logger.py:12-129)."""
from __future__ import annotations

import logging
import math
import sys
import time
from datetime import timedelta
from typing import Optional

from .distributed import get_global_rank, get_is_slurm_job


class LogFormatter(logging.Formatter):
    def __init__(self):
        super().__init__()
        self.start_time = time.time()
        self.rank = get_global_rank()
        self.show_rank = not get_is_slurm_job()  # srun --label already prints the task id

    def _prefix(self, record: logging.LogRecord) -> str:
        frac, sec = math.modf(record.created)
        stamp = time.strftime("%y-%m-%d %H:%M:%S", time.localtime(sec)) + f".{int(frac * 1_000_000):06d}"
        elapsed = timedelta(seconds=round(record.created - self.start_time))
        head = f"{self.rank}: " if self.show_rank else ""
        return f"{head}{record.levelname:<7} {stamp} - {elapsed} - "

    def format(self, record: logging.LogRecord) -> str:
        prefix = self._prefix(record)
        indent = " " * len(prefix)
        parts = [record.getMessage()]
        if record.exc_info and not record.exc_text:
            record.exc_text = self.formatException(record.exc_info)
        if record.exc_text:
            parts.append(record.exc_text)
        if record.stack_info:
            parts.append(self.formatStack(record.stack_info))
        body = "\n".join(p.rstrip("\n") for p in parts)
        return prefix + body.replace("\n", "\n" + indent)


def set_root_log_level(log_level: str) -> None:
    logger = logging.getLogger()
    level = log_level.upper()
    try:
        level = int(log_level)
    except ValueError:
        pass
    try:
        logger.setLevel(level)
    except Exception:
        logger.warning(f"Failed to set logging level to {log_level}, using default 'NOTSET'")
        logger.setLevel(logging.NOTSET)


def init_logger(log_file: Optional[str] = None, *, name: Optional[str] = None, level: str = "NOTSET") -> None:
    set_root_log_level(level)
    logger = logging.getLogger(name)
    out = logging.StreamHandler(sys.stdout)
    out.setLevel(logging.NOTSET)
    out.setFormatter(LogFormatter())
    err = logging.StreamHandler(sys.stderr)
    err.setLevel(logging.WARNING)
    err.setFormatter(LogFormatter())
    logger.handlers.clear()
    logger.handlers.extend([out, err])
    if log_file is not None and get_global_rank() == 0:
        fh = logging.FileHandler(str(log_file), "a")
        fh.setLevel(logging.NOTSET)
        fh.setFormatter(LogFormatter())
        logging.getLogger().addHandler(fh)
