"""One rule/score call per trajectory. Parity target: ``.../reward_manager/naive.py``."""
from __future__ import annotations

from .base import RewardManagerBase
from .registry import register

__all__ = ["NaiveRewardManager"]


@register("naive")
class NaiveRewardManager(RewardManagerBase):
    async def run_single(self, data):
        ids, n, source, gt, extra, item = self._unpack(data)
        extra.setdefault("num_turns", item.non_tensor_batch.get("__num_turns__"))
        if "prompts" in item.batch.keys():
            extra.setdefault("prompt_ids", item.batch["prompts"])
        extra.setdefault("response_ids", ids)
        res = await self._score(data_source=source, solution_str=self._decode(ids), ground_truth=gt, extra_info=extra)
        if isinstance(res, dict):
            return {"reward_score": float(res["score"]), "reward_extra_info": dict(res)}
        return {"reward_score": float(res), "reward_extra_info": {"acc": float(res)}}
