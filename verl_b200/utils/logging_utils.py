"""Logging set-up shared by the entry points.

Parity target: ``verl/utils/logging_utils.py`` (``configure_verl_logging`` :22, ``set_basic_config`` :35, ``log_to_file``
:42). The level comes from ``VERL_LOGGING_LEVEL`` (default WARNING).
"""

from __future__ import annotations

import logging
import os

__all__ = ["configure_verl_logging", "set_basic_config", "log_to_file"]

_PACKAGE = __name__.split(".")[0]


def configure_verl_logging() -> None:
    level = os.environ.get("VERL_LOGGING_LEVEL", "WARNING").upper()
    logger = logging.getLogger(_PACKAGE)
    logger.setLevel(getattr(logging, level, logging.WARNING))
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
        logger.addHandler(h)
        logger.propagate = False


def set_basic_config(level) -> None:
    logging.basicConfig(format="%(levelname)s:%(asctime)s:%(message)s", level=level)


def log_to_file(string: str) -> None:
    """Append one line to the file named by ``VERL_LOG_FILE`` (no-op when unset): for ranks whose stdout is not kept."""
    path = os.environ.get("VERL_LOG_FILE")
    if path:
        with open(path, "a") as f:
            f.write(string.rstrip("\n") + "\n")
