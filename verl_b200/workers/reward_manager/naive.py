"""Per-sample rule reward placed on the last valid response token.

Parity target: ``verl/workers/reward_manager/naive.py`` (175 lines) and ``batch.py`` / ``dapo.py``.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Any

import numpy as np
import torch

from ...protocol import DataProto
from ...utils.reward_score import default_compute_score
from .abstract import AbstractRewardManager
from .registry import register

__all__ = ["NaiveRewardManager", "BatchRewardManager", "DAPORewardManager", "TokenRuleRewardManager"]


def _decode(tokenizer, ids):
    return tokenizer.decode(ids, skip_special_tokens=True) if tokenizer is not None else " ".join(map(str, ids.tolist()))


def _split(item_batch, R):
    prompt = item_batch["prompts"]
    P = prompt.shape[-1]
    am = item_batch["attention_mask"]
    vp = int(am[:P].sum())
    vr = int(am[P:].sum())
    return prompt[-vp:] if vp else prompt[:0], item_batch["responses"][:vr], vr


@register("naive")
class NaiveRewardManager(AbstractRewardManager):
    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source", **kwargs):
        self.tokenizer, self.num_examine = tokenizer, num_examine
        self.compute_score = compute_score or default_compute_score
        self.reward_fn_key = reward_fn_key

    def __call__(self, data: DataProto, return_dict: bool = False):
        hit = self._extract_reward_from_rm_scores(data, return_dict)
        if hit is not None:
            return hit
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        extra = defaultdict(list)
        printed: dict[str, int] = {}
        host = data.batch.cpu() if data.batch.device is not None and data.batch.device.type != "cpu" else data.batch
        R = host["responses"].shape[-1]
        for i in range(len(data)):
            row = {k: host[k][i] for k in ("prompts", "responses", "attention_mask")}
            p_ids, r_ids, vr = _split(row, R)
            prompt_str, resp_str = _decode(self.tokenizer, p_ids), _decode(self.tokenizer, r_ids)
            rm = data.non_tensor_batch["reward_model"][i] if "reward_model" in data.non_tensor_batch else {}
            gt = rm.get("ground_truth") if isinstance(rm, dict) else None
            src = data.non_tensor_batch[self.reward_fn_key][i] if self.reward_fn_key in data.non_tensor_batch else "unknown"
            ei = data.non_tensor_batch["extra_info"][i] if "extra_info" in data.non_tensor_batch else None
            res = self.compute_score(data_source=src, solution_str=resp_str, ground_truth=gt, extra_info=ei)
            if isinstance(res, dict):
                score = res["score"]
                for k, v in res.items():
                    extra[k].append(v)
            else:
                score = res
            if vr > 0:
                reward[i, vr - 1] = float(score)
            if printed.get(src, 0) < self.num_examine:
                printed[src] = printed.get(src, 0) + 1
                print("[prompt]", prompt_str, "\n[response]", resp_str, "\n[ground_truth]", gt, "\n[score]", score)
        return {"reward_tensor": reward, "reward_extra_info": dict(extra)} if return_dict else reward


@register("batch")
class BatchRewardManager(NaiveRewardManager):
    """``compute_score`` receives whole lists (data_sources, solution_strs, ground_truths, extra_infos)."""

    def __call__(self, data: DataProto, return_dict: bool = False):
        hit = self._extract_reward_from_rm_scores(data, return_dict)
        if hit is not None:
            return hit
        host = data.batch.cpu() if data.batch.device is not None and data.batch.device.type != "cpu" else data.batch
        R = host["responses"].shape[-1]
        strs, lens = [], []
        for i in range(len(data)):
            _, r_ids, vr = _split({k: host[k][i] for k in ("prompts", "responses", "attention_mask")}, R)
            strs.append(_decode(self.tokenizer, r_ids))
            lens.append(vr)
        gts = [rm.get("ground_truth") if isinstance(rm, dict) else None for rm in data.non_tensor_batch.get("reward_model", [{}] * len(data))]
        srcs = list(data.non_tensor_batch.get(self.reward_fn_key, ["unknown"] * len(data)))
        eis = list(data.non_tensor_batch.get("extra_info", [None] * len(data)))
        scores = self.compute_score(data_sources=srcs, solution_strs=strs, ground_truths=gts, extra_infos=eis)
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        extra = defaultdict(list)
        for i, s in enumerate(scores):
            if isinstance(s, dict):
                for k, v in s.items():
                    extra[k].append(v)
                s = s["score"]
            if lens[i] > 0:
                reward[i, lens[i] - 1] = float(s)
        return {"reward_tensor": reward, "reward_extra_info": dict(extra)} if return_dict else reward


@register("dapo")
class DAPORewardManager(NaiveRewardManager):
    """Naive rule reward plus the DAPO soft over-length penalty."""

    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source",
                 max_resp_len=None, overlong_buffer_cfg=None, **kwargs):
        super().__init__(tokenizer, num_examine, compute_score, reward_fn_key)
        self.max_resp_len, self.buf = max_resp_len, overlong_buffer_cfg
        if self.buf is not None:
            assert max_resp_len is not None, "max_resp_len must be provided if overlong_buffer_cfg is set"

    def __call__(self, data: DataProto, return_dict: bool = False):
        out = super().__call__(data, return_dict=True)
        reward, extra = out["reward_tensor"], out["reward_extra_info"]
        if self.buf is not None and self.buf.get("enable", False):
            L = int(self.buf["len"])
            expected = self.max_resp_len - L
            lens = data.batch["response_mask"].sum(-1) if "response_mask" in data.batch.keys() else \
                data.batch["attention_mask"][:, -reward.shape[1]:].sum(-1)
            pen = torch.clamp(-(lens.float() - expected) / L * float(self.buf["penalty_factor"]), max=0.0)
            for i in range(reward.shape[0]):
                n = int(lens[i])
                if n > 0:
                    reward[i, n - 1] += pen[i].item()
            if self.buf.get("log", False):
                extra["overlong_reward"] = pen.tolist()
                extra["overlong"] = (pen < 0).tolist()
        return {"reward_tensor": reward, "reward_extra_info": extra} if return_dict else reward


@register("token_rule")
class TokenRuleRewardManager(AbstractRewardManager):
    """Synthetic token-level rule evaluated on the device without a tokenizer: the score of a sample is the
    fraction of its response tokens whose id is congruent to the prompt's first token id modulo ``modulus``.
    ``placement='last'`` puts the scalar on the final valid response token."""

    def __init__(self, tokenizer=None, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source",
                 modulus: int = 7, placement: str = "last", **kwargs):
        self.modulus, self.placement = int(modulus), placement

    def __call__(self, data: DataProto, return_dict: bool = False):
        b = data.batch
        resp = b["responses"]
        mask = (b["response_mask"] if "response_mask" in b.keys() else b["attention_mask"][:, -resp.shape[1]:]).to(torch.float32)
        prompts, pm = b["prompts"], b["attention_mask"][:, : b["prompts"].shape[1]]
        first_col = torch.argmax(pm.to(torch.int32), dim=1, keepdim=True)
        first = torch.gather(prompts, 1, first_col)
        hit = ((resp % self.modulus) == (first % self.modulus)).to(torch.float32) * mask
        n = mask.sum(-1)
        score = hit.sum(-1) / n.clamp(min=1)
        reward = torch.zeros_like(mask)
        last = (n.long() - 1).clamp(min=0)
        reward.scatter_(1, last.unsqueeze(1), (score * (n > 0)).unsqueeze(1))
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": {"acc": score.detach().cpu().tolist()}}
        return reward
