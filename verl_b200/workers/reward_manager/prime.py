"""Reward manager that scores all samples of a batch in parallel worker processes with a per-sample time limit (code
execution and heavy verifiers must not stall the training loop); a sample whose scorer fails or runs out of time scores 0.

Parity target: ``verl/workers/reward_manager/prime.py`` (``single_compute_score`` :31, ``parallel_compute_score_async``
:45, ``run_reward_scoring`` :91, ``PrimeRewardManager`` :103).
"""

from __future__ import annotations

import asyncio
from concurrent.futures import ProcessPoolExecutor
from functools import partial
from typing import Any, Callable, Optional

import torch

from ...protocol import DataProto
from ...utils.reward_score import default_compute_score
from .abstract import AbstractRewardManager
from .registry import register

__all__ = ["PrimeRewardManager", "run_reward_scoring", "parallel_compute_score_async", "single_compute_score"]


async def single_compute_score(evaluation_func: Callable, completion, reference, task, task_extra_info, executor, timeout: float = 300.0):
    loop = asyncio.get_running_loop()
    try:
        fut = loop.run_in_executor(executor, partial(evaluation_func, task, completion, reference, task_extra_info))
        return await asyncio.wait_for(fut, timeout=timeout)
    except asyncio.TimeoutError:
        return None
    except Exception:
        return None


async def parallel_compute_score_async(evaluation_func: Callable, completions: list, references: list, tasks: list,
                                       extra_info: Optional[list] = None, num_processes: int = 64, timeout: float = 300.0) -> list[float]:
    extra_info = extra_info if extra_info is not None else [None] * len(tasks)
    with ProcessPoolExecutor(max_workers=max(1, min(num_processes, len(tasks) or 1))) as ex:
        try:
            results = await asyncio.gather(*[single_compute_score(evaluation_func, c, r, t, e, ex, timeout)
                                             for c, r, t, e in zip(completions, references, tasks, extra_info)])
        finally:
            for p in list(getattr(ex, "_processes", {}).values()):  # stragglers past their time limit
                if p.is_alive():
                    p.terminate()
    out = []
    for r in results:
        if r is None:
            out.append(0.0)
        elif isinstance(r, dict):
            out.append(float(r.get("score", 0.0)))
        elif isinstance(r, (tuple, list)):
            out.append(float(r[0]))
        else:
            out.append(float(r))
    return out


def run_reward_scoring(evaluation_func: Callable, completions: list, references: list, tasks: list, extra_info: Optional[list] = None,
                       num_processes: int = 64, timeout: float = 300.0) -> list[float]:
    loop = asyncio.new_event_loop()
    try:
        return loop.run_until_complete(parallel_compute_score_async(evaluation_func, completions, references, tasks, extra_info,
                                                                    num_processes, timeout))
    finally:
        loop.close()


@register("prime")
class PrimeRewardManager(AbstractRewardManager):
    def __init__(self, tokenizer, num_examine: int = 0, compute_score: Optional[Callable] = None, reward_fn_key: str = "data_source",
                 num_processes: int = 64, timeout: float = 300.0, **kwargs):
        self.tokenizer, self.num_examine = tokenizer, num_examine
        self.compute_score = compute_score or default_compute_score
        self.reward_fn_key, self.num_processes, self.timeout = reward_fn_key, int(num_processes), float(timeout)

    def _decode(self, ids) -> str:
        return self.tokenizer.decode(ids, skip_special_tokens=True) if self.tokenizer is not None else " ".join(map(str, ids.tolist()))

    def verify(self, data: DataProto) -> list[float]:
        """Scores of all rows; also stored as ``data.batch["acc"]``."""
        resp = data.batch["responses"].cpu()
        R = resp.shape[-1]
        valid = data.batch["attention_mask"][:, -R:].sum(-1).cpu().tolist()
        texts = [self._decode(resp[i, : int(valid[i])]) for i in range(len(data))]
        nt = data.non_tensor_batch
        gts = [(rm.get("ground_truth") if isinstance(rm, dict) else None) for rm in nt["reward_model"]] if "reward_model" in nt else [None] * len(data)
        srcs = list(nt[self.reward_fn_key]) if self.reward_fn_key in nt else ["unknown"] * len(data)
        extra = list(nt["extra_info"]) if "extra_info" in nt else None
        scores = run_reward_scoring(self.compute_score, texts, gts, srcs, extra, self.num_processes, self.timeout)
        data.batch["acc"] = torch.tensor(scores, dtype=torch.float32, device=data.batch["responses"].device)
        return scores

    def __call__(self, data: DataProto, return_dict: bool = False) -> Any:
        hit = self._extract_reward_from_rm_scores(data, return_dict)
        if hit is not None:
            return hit
        scores = self.verify(data)
        R = data.batch["responses"].shape[-1]
        valid = data.batch["attention_mask"][:, -R:].sum(-1)
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        for i, s in enumerate(scores):
            if int(valid[i]) > 0:
                reward[i, int(valid[i]) - 1] = s
        return {"reward_tensor": reward, "reward_extra_info": {"acc": scores}} if return_dict else reward
