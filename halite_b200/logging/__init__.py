"""Rank-aware logging (reference: logging/__init__.py:6-20, logging/logger.py:25-198)."""

from .logger import DistributedLogger, get_logger, logger

__all__ = ["DistributedLogger", "get_logger", "logger"]
