"""Console / file loggers (parity: ``physicsnemo/utils/logging/console.py:23-91``)."""
import logging
import os
import sys


def _color(text: str, code: str) -> str:
    if os.environ.get("NO_COLOR") or not (sys.stdout.isatty() or os.environ.get("FORCE_COLOR")):
        return text
    return f"\033[{code}m{text}\033[0m"


class PythonLogger:
    """Simple console logger with optional file output and coloured ``success`` / ``warning`` / ``error``."""

    def __init__(self, name: str = "launch"):
        self.logger = logging.getLogger(name)
        self.logger.handlers.clear()
        fmt = logging.Formatter("[%(asctime)s - %(name)s - %(levelname)s] %(message)s", datefmt="%H:%M:%S")
        handler = logging.StreamHandler()
        handler.setFormatter(fmt)
        handler.setLevel(logging.DEBUG)
        self.logger.addHandler(handler)
        self.logger.setLevel(logging.DEBUG)
        self.logger.propagate = False
        self._fmt = fmt

    def file_logging(self, file_name: str = "launch.log"):
        if os.path.exists(file_name):
            try:
                os.remove(file_name)
            except FileNotFoundError:
                pass
        fh = logging.FileHandler(file_name, mode="a+", encoding="utf-8")
        fh.setFormatter(self._fmt)
        fh.setLevel(logging.DEBUG)
        self.logger.addHandler(fh)

    def log(self, message: str):
        self.logger.info(message)

    def info(self, message: str):
        self.logger.info(_color(message, "94"))

    def success(self, message: str):
        self.logger.info(_color(message, "92"))

    def warning(self, message: str):
        self.logger.warning(_color(message, "93"))

    def error(self, message: str):
        self.logger.error(_color(message, "91"))


class RankZeroLoggingWrapper:
    """Forwards logging calls on rank 0 only; other ranks get no-ops."""

    def __init__(self, obj, dist):
        self.obj, self.dist = obj, dist

    def __getattr__(self, name):
        attr = getattr(self.obj, name)
        if callable(attr):
            def wrapper(*args, **kwargs):
                if self.dist.rank == 0:
                    return attr(*args, **kwargs)
                return None

            return wrapper
        return attr
