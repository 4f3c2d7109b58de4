"""GDPO: keeps every named component of a dict-valued score so that the advantage estimator can normalise the
components separately. Parity target: ``.../reward_manager/gdpo.py``."""
from __future__ import annotations

from .naive import NaiveRewardManager
from .registry import register

__all__ = ["GDPORewardManager"]


@register("gdpo")
class GDPORewardManager(NaiveRewardManager):
    async def run_single(self, data):
        out = await super().run_single(data)
        info = out["reward_extra_info"]
        comps = {k: float(v) for k, v in info.items() if k != "score" and isinstance(v, (int, float, bool))}
        info["reward_components"] = comps
        return out
