"""`get_logger(mesh)` returns a logger that prints on selected ranks only and prefixes each
message with the caller's `file:line function()`. Handlers: rich (when importable and a
terminal is attached), ANSI colour, or plain."""

from __future__ import annotations

import inspect
import logging
import os
import sys

try:  # rich is optional
    from rich.logging import RichHandler
except Exception:  # pragma: no cover
    RichHandler = None

_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m",
           "CRITICAL": "\033[35m"}


class _ColorFormatter(logging.Formatter):
    def format(self, record):
        msg = super().format(record)
        c = _COLORS.get(record.levelname)
        return f"{c}{msg}\033[0m" if c and sys.stderr.isatty() else msg


def _make_handler(mode):
    if mode == "rich" and RichHandler is not None:
        return RichHandler(show_path=False, keywords=["epoch", "loss", "lr", "step", "grad norm"])
    h = logging.StreamHandler()
    fmt = "[%(asctime)s] %(levelname)s %(message)s"
    h.setFormatter(_ColorFormatter(fmt, "%H:%M:%S") if mode == "color" else logging.Formatter(fmt, "%H:%M:%S"))
    return h


class DistributedLogger:
    """Wraps a `logging.Logger`; a call prints only when this process's rank is in `ranks`
    (global ranks by default, or ranks within a mesh dimension via `ranks={"dp": (0,)}`)."""

    def __init__(self, name="halite_b200", mesh=None, mode="rich", level=logging.INFO, ranks=(0,)):
        self.logger = logging.getLogger(name)
        self.logger.propagate = False
        if not self.logger.handlers:
            self.logger.addHandler(_make_handler(mode))
        self.logger.setLevel(level)
        self.mesh = mesh
        self.ranks = ranks

    def _rank(self):
        try:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                return dist.get_rank()
        except Exception:
            pass
        return int(os.environ.get("RANK", "0"))

    def _enabled(self, ranks):
        ranks = self.ranks if ranks is None else ranks
        if ranks is None or ranks == "all":
            return True
        if isinstance(ranks, dict):
            if self.mesh is None:
                return True
            return all(self.mesh.local_rank_in(dim) in allowed for dim, allowed in ranks.items())
        return self._rank() in tuple(ranks)

    def _log(self, level, msg, ranks=None, stacklevel=2):
        if not self._enabled(ranks):
            return
        frame = inspect.stack()[stacklevel]
        where = f"FROM {os.path.basename(frame.filename)}:{frame.lineno} {frame.function}()"
        self.logger.log(level, f"{where} {msg}")

    def debug(self, msg, ranks=None):
        self._log(logging.DEBUG, msg, ranks)

    def info(self, msg, ranks=None):
        self._log(logging.INFO, msg, ranks)

    def warning(self, msg, ranks=None):
        self._log(logging.WARNING, msg, ranks)

    def error(self, msg, ranks=None):
        self._log(logging.ERROR, msg, ranks)

    def setLevel(self, level):
        self.logger.setLevel(level)


_default = None


def get_logger(mesh=None, mode="rich", name="halite_b200", ranks=(0,)):
    global _default
    _default = DistributedLogger(name, mesh, mode, ranks=ranks)
    return _default


class _Proxy:
    """Module-level `logger` that follows the most recent `get_logger` call."""

    def __getattr__(self, item):
        global _default
        if _default is None:
            _default = DistributedLogger(mode="plain")
        return getattr(_default, item)


logger = _Proxy()
