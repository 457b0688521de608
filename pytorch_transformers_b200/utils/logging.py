"""One logger namespace for the library, with its level from the environment.

Every module logs under ``pytorch_transformers_b200``; the library's root logger gets one
stream handler (stderr) and does not propagate, and ``PTB200_VERBOSITY`` (debug, info, warning,
error, critical) sets the level, default warning — what ``TRANSFORMERS_VERBOSITY`` does for the
reference (src/transformers/utils/logging.py:44-77, 84-109, 147-158). Messages about compiling
the kernels are ``info`` records that are shown at the default level too (``always``): a first
call in a fresh checkout takes a minute and must not look hung.
"""
from __future__ import annotations

import logging
import os
import sys
import threading
from typing import Optional

LIBRARY = "pytorch_transformers_b200"
ENV = "PTB200_VERBOSITY"
log_levels = {"debug": logging.DEBUG, "info": logging.INFO, "warning": logging.WARNING, "error": logging.ERROR,
              "critical": logging.CRITICAL}
_default_level = logging.WARNING
_lock = threading.Lock()
_handler: Optional[logging.Handler] = None


def _level_from_env() -> int:
    name = os.getenv(ENV)
    if name:
        if name.lower() in log_levels:
            return log_levels[name.lower()]
        logging.getLogger().warning(f"unknown {ENV}={name}; one of: {', '.join(log_levels)}")
    return _default_level


class _StderrHandler(logging.StreamHandler):
    """Writes to whatever sys.stderr is when the record is emitted (tests swap it)."""

    def __init__(self):
        super().__init__(sys.stderr)

    def emit(self, record):
        self.stream = sys.stderr
        super().emit(record)


def _configure() -> None:
    global _handler
    with _lock:
        if _handler is not None:
            return
        _handler = _StderrHandler()
        _handler.setFormatter(logging.Formatter("[%(name)s] %(message)s"))
        root = logging.getLogger(LIBRARY)
        root.addHandler(_handler)
        root.setLevel(_level_from_env())
        root.propagate = False


def get_logger(name: Optional[str] = None) -> logging.Logger:
    """The logger ``name`` (a module's ``__name__``) under the library's namespace."""
    _configure()
    if not name:
        return logging.getLogger(LIBRARY)
    return logging.getLogger(name if name.startswith(LIBRARY) else f"{LIBRARY}.{name}")


def set_verbosity(level) -> None:
    _configure()
    logging.getLogger(LIBRARY).setLevel(log_levels[level.lower()] if isinstance(level, str) else int(level))


def get_verbosity() -> int:
    _configure()
    return logging.getLogger(LIBRARY).getEffectiveLevel()


def always(logger: logging.Logger, message: str) -> None:
    """A progress line that is shown unless the level is above warning (compilation at first use)."""
    logger.log(logging.WARNING if logger.getEffectiveLevel() <= logging.WARNING else logging.INFO, message)
