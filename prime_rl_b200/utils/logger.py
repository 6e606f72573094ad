"""Process-wide logger (loguru) with an optional JSON sink and stdlib interception."""

from __future__ import annotations

import logging
import sys
from pathlib import Path

from loguru import logger as _logger

_configured = False


class _Intercept(logging.Handler):
    def emit(self, record: logging.LogRecord) -> None:
        try:
            level = _logger.level(record.levelname).name
        except ValueError:
            level = record.levelno
        _logger.opt(depth=6, exception=record.exc_info).log(level, record.getMessage())


def _arm_stack_dumps() -> None:
    import faulthandler
    import signal

    try:
        faulthandler.enable(file=sys.stderr, all_threads=True)
        if hasattr(signal, "SIGUSR1"):
            faulthandler.register(signal.SIGUSR1, file=sys.stderr, all_threads=True, chain=False)
    except (ValueError, OSError, AttributeError):      # no usable stderr (embedded interpreters, closed streams)
        pass


def setup_logger(level: str = "info", *, log_file: Path | None = None, json_logging: bool = False,
                 tag: str | None = None, intercept_stdlib: bool = False):
    """(Re)configures the global logger: console sink, optional per-process log file. Also arms the stack dumps:
    a native crash prints the Python stacks, and ``kill -USR1 <pid>`` prints them from a process that seems stuck."""
    global _configured
    _arm_stack_dumps()
    _logger.remove()
    prefix = f"[{tag}] " if tag else ""
    fmt = "<dim>{time:HH:mm:ss}</dim> <level>{level: <7}</level> " + prefix + "{message}"
    if json_logging:
        _logger.add(sys.stdout, level=level.upper(), serialize=True)
    else:
        _logger.add(sys.stdout, level=level.upper(), format=fmt, colorize=False)
    if log_file is not None:
        log_file.parent.mkdir(parents=True, exist_ok=True)
        _logger.add(str(log_file), level=level.upper(), format=fmt, serialize=json_logging)
    if intercept_stdlib:
        logging.basicConfig(handlers=[_Intercept()], level=0, force=True)
    _configured = True
    return _logger


def get_logger():
    if not _configured:
        setup_logger()
    return _logger


def reset_logger() -> None:
    global _configured
    _logger.remove()
    _configured = False
