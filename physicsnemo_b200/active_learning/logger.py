"""Structured logging for active-learning runs: console lines with context tags, JSON lines on disk.

Parity: ``physicsnemo/active_learning/logger.py`` (``ActiveLearningLoggerAdapter``, ``JSONFormatter``,
``ContextFormatter``, ``ContextInjectingFilter``, ``setup_active_learning_logger``, ``log_context``).
Console colouring uses plain ANSI escapes (no third-party colour package) and is applied only
when the stream is a terminal.
"""
from __future__ import annotations

import json
import logging
import sys
from contextlib import contextmanager
from datetime import datetime
from pathlib import Path
from threading import local
from typing import Any

_context_storage = local()
_ANSI = {"red": "31", "yellow": "33", "white": "37", "cyan": "36", "blue": "34"}
_STANDARD_RECORD_KEYS = set(logging.LogRecord("", 0, "", 0, "", (), None).__dict__) | {"message", "asctime"}


def _paint(text: str, colour: str, enabled: bool) -> str:
    return f"\033[{_ANSI[colour]}m{text}\033[0m" if enabled else text


def _get_context_stack() -> list:
    if not hasattr(_context_storage, "context_stack"):
        _context_storage.context_stack = []
    return _context_storage.context_stack


class ActiveLearningLoggerAdapter(logging.LoggerAdapter):
    """Adds the driver's step index, run id and phase to every record."""

    def __init__(self, logger: logging.Logger, driver_ref: Any = None):
        super().__init__(logger, {})
        self.driver_ref = driver_ref

    def process(self, msg, kwargs):
        if self.driver_ref is not None:
            extra = kwargs.get("extra", {})
            for key, attr in (("iteration", "active_learning_step_idx"), ("run_id", "run_id"), ("phase", "current_phase")):
                value = getattr(self.driver_ref, attr, None)
                if value is not None:
                    extra[key] = str(value) if key == "phase" else value
            if extra:
                kwargs["extra"] = extra
        return msg, kwargs


class JSONFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        entry = {
            "timestamp": datetime.fromtimestamp(record.created).isoformat(),
            "level": record.levelname, "logger": record.name, "message": record.getMessage(),
            "module": record.module, "function": record.funcName, "line": record.lineno,
        }
        for key, value in record.__dict__.items():
            if key not in _STANDARD_RECORD_KEYS and key not in entry:
                entry[key] = value
        return json.dumps(entry, default=str)


class ContextFormatter(logging.Formatter):
    _LEVEL_COLOURS = ((logging.ERROR, "red"), (logging.WARNING, "yellow"), (logging.INFO, "white"), (0, "cyan"))

    def __init__(self, fmt=None, colour: bool | None = None):
        super().__init__(fmt)
        self.colour = sys.stderr.isatty() if colour is None else colour

    def format(self, record):
        tags = []
        for label, attr in (("obj", "caller_object"), ("run", "run_id"), ("iter", "iteration"), ("phase", "phase")):
            value = getattr(record, attr, None)
            if value is not None and value != "":
                tags.append(f"{label}:{value}")
        tags += [f"{k}:{v}" for k, v in (getattr(record, "context", None) or {}).items()]
        colour = next(c for lvl, c in self._LEVEL_COLOURS if record.levelno >= lvl)
        msg = _paint(super().format(record), colour, self.colour)
        return msg + (" " + _paint(f"[{', '.join(tags)}]", "blue", self.colour) if tags else "")


class ContextInjectingFilter(logging.Filter):
    def filter(self, record):
        stack = _get_context_stack()
        if stack:
            top = stack[-1]
            if top["caller_object"]:
                record.caller_object = top["caller_object"]
            if top["iteration"] is not None:
                record.iteration = top["iteration"]
            if top.get("phase"):
                record.phase = top["phase"]
            if top["context"]:
                record.context = top["context"]
        return True


def setup_active_learning_logger(name: str, run_id: str, log_dir: str | Path = Path("active_learning_logs"),
                                 level: int = logging.INFO) -> logging.Logger:
    logger = logging.getLogger(name)
    logger.setLevel(level)
    for h in list(logger.handlers):
        logger.removeHandler(h)
        h.close()
    logger.propagate = False
    log_dir = Path(log_dir)
    log_dir.mkdir(parents=True, exist_ok=True)
    console = logging.StreamHandler()
    console.setLevel(logging.DEBUG)
    console.setFormatter(ContextFormatter("%(asctime)s - %(name)s - %(levelname)s - %(message)s"))
    console.addFilter(ContextInjectingFilter())
    logger.addHandler(console)
    file_handler = logging.FileHandler(log_dir / f"{run_id}.log", mode="w")
    file_handler.setLevel(logging.DEBUG)
    file_handler.setFormatter(JSONFormatter())
    file_handler.addFilter(ContextInjectingFilter())
    logger.addHandler(file_handler)
    return logger


@contextmanager
def log_context(caller_object: str | None = None, iteration: int | None = None, phase: str | None = None, **kwargs: Any):
    stack = _get_context_stack()
    stack.append({"caller_object": caller_object, "iteration": iteration, "phase": phase, "context": kwargs})
    try:
        yield
    finally:
        stack.pop()
