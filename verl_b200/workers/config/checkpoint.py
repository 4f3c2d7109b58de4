"""Checkpoint content flags. Parity target: ``verl/workers/config/checkpoint.py`` (49 lines)."""

from __future__ import annotations

from dataclasses import dataclass, field

from ...base_config import BaseConfig

__all__ = ["CheckpointConfig"]


@dataclass
class CheckpointConfig(BaseConfig):
    save_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    load_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    async_save: bool = False
    mbridge_config: dict = field(default_factory=dict)
