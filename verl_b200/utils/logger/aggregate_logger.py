"""Console logger of step metrics and rank-aware print helpers.

Parity target: ``verl/utils/logger/aggregate_logger.py`` (``concat_dict_to_str`` :26, ``LocalLogger`` :35,
``DecoratorLoggerBase`` :54, ``print_rank_0`` :89, ``print_with_rank`` :98, ``print_with_rank_and_timer`` :112,
``log_with_rank`` :128).
"""

from __future__ import annotations

import datetime
import logging
import numbers
from typing import Optional

import torch.distributed as dist

__all__ = ["concat_dict_to_str", "LocalLogger", "DecoratorLoggerBase", "print_rank_0", "print_with_rank",
           "print_with_rank_and_timer", "log_with_rank"]


def concat_dict_to_str(dict: dict, step) -> str:
    parts = [f"step:{step}"]
    for k, v in dict.items():
        if isinstance(v, numbers.Number):
            parts.append(f"{k}:{v:.3f}")
    return " - ".join(parts)


class LocalLogger:
    """The ``console`` tracking backend: one line of numeric metrics per step."""

    def __init__(self, print_to_console: bool = True):
        self.print_to_console = print_to_console

    def flush(self) -> None:
        pass

    def log(self, data: dict, step) -> None:
        if self.print_to_console:
            print(concat_dict_to_str(data, step), flush=True)


class DecoratorLoggerBase:
    """Base of decorators that report (timings, memory, ...) either by ``print`` or through a ``logging.Logger``."""

    def __init__(self, role: str, logger: Optional[logging.Logger] = None, level=logging.DEBUG, rank: int = 0,
                 log_only_rank_0: bool = True):
        self.role, self.logger, self.level, self.rank, self.log_only_rank_0 = role, logger, level, rank, log_only_rank_0
        self.logging_function = self.log_by_print if logger is None else self.log_by_logging

    def log_by_print(self, log_str: str) -> None:
        if not self.log_only_rank_0 or self.rank == 0:
            print(f"{self.role} {log_str}", flush=True)

    def log_by_logging(self, log_str: str) -> None:
        if not self.log_only_rank_0 or self.rank == 0:
            self.logger.log(self.level, f"{self.role} {log_str}")


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def print_rank_0(message) -> None:
    if _rank() == 0:
        print(message, flush=True)


def print_with_rank(message: str, rank: int = 0, log_only_rank_0: bool = False) -> None:
    if not log_only_rank_0 or rank == 0:
        print(f"[Rank {rank}] {message}", flush=True)


def print_with_rank_and_timer(message: str, rank: int = 0, log_only_rank_0: bool = False) -> None:
    if not log_only_rank_0 or rank == 0:
        now = datetime.datetime.now().strftime("%Y-%m-%d %H:%M:%S")
        print(f"[{now}] [Rank {rank}] {message}", flush=True)


def log_with_rank(message: str, rank, logger: logging.Logger, level=logging.INFO, log_only_rank_0: bool = False) -> None:
    if not log_only_rank_0 or rank == 0:
        logger.log(level, f"[Rank {rank}] {message}")
