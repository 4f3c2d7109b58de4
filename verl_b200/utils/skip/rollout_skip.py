"""Rollout skipping: ``generate_sequences`` results are stored per step under
``<dump_dir>/<project>/<experiment>/step_<N>/gen_batch.pkl``; a later run with the same prompts loads them instead of
generating. ``action_on_miss`` = ``generate`` (default: generate and dump) or ``latest`` (replay the closest earlier
step, for quick smoke runs). ``max_dump_step`` bounds how many steps are written.

Parity target: ``verl/utils/skip/rollout_skip.py:26-165`` (``RolloutSkip``); the TransferQueue and async variants
(:166-497) key dumps by prompt uid / sample id and are covered by ``uid_key``.
"""

from __future__ import annotations

import os
import re
from pathlib import Path
from typing import Callable

from ...protocol import DataProto
from .skip_manager import BaseSkip, register_skip

__all__ = ["RolloutSkip", "parse_async_rollout_sample_step"]


def _g(cfg, key, default=None):
    if cfg is None:
        return default
    v = cfg.get(key, default) if hasattr(cfg, "get") else getattr(cfg, key, default)
    return default if v is None else v


def parse_async_rollout_sample_step(sample_id: str) -> int:
    """``"<uid>@<version>"`` -> version (the weight version a streamed sample was started under)."""
    m = re.search(r"@(\d+)$", str(sample_id))
    return int(m.group(1)) if m else -1


@register_skip("rollout")
class RolloutSkip(BaseSkip):
    def __init__(self, local_config, global_config):
        super().__init__(local_config, global_config)
        tr = _g(global_config, "trainer", {})
        self.root = Path(os.path.expanduser(str(_g(local_config, "dump_dir", "~/.verl_b200/rollout_dump"))))
        self.project, self.experiment = str(_g(tr, "project_name", "project")), str(_g(tr, "experiment_name", "run"))
        self.max_dump_step = int(_g(local_config, "max_dump_step", 1 << 30))
        self.action_on_miss = str(_g(local_config, "action_on_miss", "generate"))
        self.hits = self.misses = 0

    def _project_dir(self) -> Path:
        return self.root / self.project / self.experiment

    def _step_dir(self, step: int) -> Path:
        return self._project_dir() / f"step_{step}"

    def _valid(self, path: Path) -> bool:
        return (path / "gen_batch.pkl").exists()

    def _available_steps(self) -> list[int]:
        d = self._project_dir()
        if not d.exists():
            return []
        out = []
        for p in d.iterdir():
            m = re.fullmatch(r"step_(\d+)", p.name)
            if m and self._valid(p):
                out.append(int(m.group(1)))
        return sorted(out)

    def _resolve(self, step: int) -> int:
        if self._valid(self._step_dir(step)):
            return step
        if self.action_on_miss == "latest":
            earlier = [s for s in self._available_steps() if s <= step]
            if earlier:
                return earlier[-1]
        return -1

    def meet_precondition(self, step: int, func: Callable, *args, **kwargs) -> bool:
        ok = self._resolve(step) >= 0
        self.hits += int(ok)
        self.misses += int(not ok)
        return ok

    def warp_function(self, step: int, func: Callable, *args, **kwargs):
        return DataProto.load_from_disk(str(self._step_dir(self._resolve(step)) / "gen_batch.pkl"))

    def prepare_data(self, step: int, result, *args, **kwargs) -> None:
        if step < 0 or step > self.max_dump_step or not isinstance(result, DataProto):
            return
        d = self._step_dir(step)
        d.mkdir(parents=True, exist_ok=True)
        result.save_to_disk(str(d / "gen_batch.pkl"))
