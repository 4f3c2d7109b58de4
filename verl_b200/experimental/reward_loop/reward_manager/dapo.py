"""DAPO scoring: the rule score plus the soft over-length penalty of the last ``overlong_buffer.len`` tokens.
Parity target: ``.../reward_manager/dapo.py`` (``overlong_buffer`` :80-110)."""
from __future__ import annotations

from .naive import NaiveRewardManager
from .registry import register

__all__ = ["DAPORewardManager"]


@register("dapo")
class DAPORewardManager(NaiveRewardManager):
    def _buffer_cfg(self):
        r = self.config.get("reward") or self.config.get("reward_model") or {}
        kw = (r.get("reward_kwargs") or {}) if hasattr(r, "get") else {}
        return kw.get("overlong_buffer_cfg") or kw.get("overlong_buffer"), kw.get("max_resp_len")

    async def run_single(self, data):
        out = await super().run_single(data)
        buf, max_len = self._buffer_cfg()
        if buf and buf.get("enable", False):
            assert max_len is not None, "max_resp_len is required with the overlong buffer"
            _, n, *_ = self._unpack(data)
            L = int(buf["len"])
            expected = int(max_len) - L
            pen = min(-(n - expected) / L * float(buf["penalty_factor"]), 0.0)
            out["reward_score"] += pen
            if buf.get("log", False):
                out["reward_extra_info"].update(overlong_reward=pen, overlong=bool(pen < 0))
        return out
