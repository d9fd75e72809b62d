"""Python-side logging set-up: coloured single-line records on stderr, or plain records
when ``DD_ENV`` is set (log shippers dislike escape codes). Mirrors the behaviour of the
reference's python/pplx_garden/utils/logging_utils.py:8-84.
"""

from __future__ import annotations

import logging
import os
import sys

_COLORS = {
    logging.DEBUG: "\x1b[34m",
    logging.INFO: "\x1b[32m",
    logging.WARNING: "\x1b[33m",
    logging.ERROR: "\x1b[31m",
    logging.CRITICAL: "\x1b[41m",
}
_RESET = "\x1b[0m"


class LoggerFormatter(logging.Formatter):
    """``time LEVEL [pid] name:line message`` with the level coloured on terminals."""

    def __init__(self, color: bool = True) -> None:
        super().__init__()
        self._color = color

    def format(self, record: logging.LogRecord) -> str:
        level = record.levelname[:5].ljust(5)
        if self._color:
            level = f"{_COLORS.get(record.levelno, '')}{level}{_RESET}"
        when = self.formatTime(record, "%H:%M:%S")
        line = f"{when}.{int(record.msecs):03d} {level} [{record.process}] {record.name}:{record.lineno} {record.getMessage()}"
        if record.exc_info:
            line += "\n" + self.formatException(record.exc_info)
        return line


def setup(level: int | str = logging.INFO, *, stream=None) -> None:
    """Install one stderr handler on the root logger (idempotent)."""
    root = logging.getLogger()
    for handler in list(root.handlers):
        if getattr(handler, "_pplx_garden", False):
            root.removeHandler(handler)
    stream = stream or sys.stderr
    handler = logging.StreamHandler(stream)
    handler._pplx_garden = True  # type: ignore[attr-defined]
    plain = bool(os.environ.get("DD_ENV"))
    if plain:
        handler.setFormatter(logging.Formatter("%(asctime)s %(levelname)s [%(process)d] %(name)s:%(lineno)d %(message)s"))
    else:
        handler.setFormatter(LoggerFormatter(color=hasattr(stream, "isatty") and stream.isatty()))
    root.addHandler(handler)
    root.setLevel(level)


def get_logger(path: str) -> logging.Logger:
    return logging.getLogger(path)
