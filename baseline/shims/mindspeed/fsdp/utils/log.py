"""Rank-aware logging helpers (stand-in for the MindSpeed package's module of the same name)."""
import logging
import os

import torch.distributed as dist


def _rank() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return int(os.environ.get("RANK", "0"))


def print_rank(log_fn, message, rank=0):
    """Call ``log_fn(message)`` on one rank only (``rank=None``: on every rank)."""
    if rank is None or _rank() == rank:
        log_fn(message)


def set_log_level(level=None):
    """Root logger level from the argument or the LOG_LEVEL environment variable (default INFO)."""
    if level is None:
        level = os.environ.get("LOG_LEVEL", "INFO")
    if isinstance(level, str):
        level = getattr(logging, level.upper(), logging.INFO)
    root = logging.getLogger()
    if not root.handlers:
        logging.basicConfig(level=level, format="%(message)s")
    root.setLevel(level)
