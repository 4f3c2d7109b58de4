"""Agent-loop side of distillation: after a trajectory is sampled, ask the right teacher for top-k log-probs over
the response positions and attach them, padded to the response length, as ``teacher_ids`` / ``teacher_logprobs``.

Parity target: ``verl/experimental/teacher_loop/teacher_manager.py`` (``_get_teacher_sampling_params`` :35,
``_pad_teacher_outputs`` :59, ``AsyncTeacherLLMServerManager`` :78-141).
"""

from __future__ import annotations

from typing import Optional

import torch

from .teacher_model import MultiTeacherModelManager, TeacherModelManager

__all__ = ["AsyncTeacherLLMServerManager", "pad_teacher_outputs"]


def pad_teacher_outputs(ids: torch.Tensor, lps: torch.Tensor, response_length: int, pad_id: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """Right-pad [n, k] records to [response_length, k]; padded rows carry log-prob 0 on id ``pad_id``."""
    n, k = ids.shape
    out_i = torch.full((response_length, k), pad_id, dtype=torch.int64)
    out_l = torch.zeros(response_length, k, dtype=torch.float32)
    m = min(n, response_length)
    out_i[:m], out_l[:m] = ids[:m], lps[:m]
    return out_i, out_l


class AsyncTeacherLLMServerManager:
    def __init__(self, teachers: MultiTeacherModelManager | TeacherModelManager, response_length: int, pad_token_id: int = 0):
        self.teachers = teachers if isinstance(teachers, MultiTeacherModelManager) else MultiTeacherModelManager({teachers.name: teachers})
        self.response_length, self.pad_token_id = int(response_length), int(pad_token_id)

    def _resolve_teacher_key(self, routing_key: Optional[str]) -> str:
        return str(routing_key) if routing_key is not None and str(routing_key) in self.teachers.managers else self.teachers.default

    async def compute_teacher_logprobs(self, request_id: str, prompt_ids: list[int], response_ids: list[int],
                                       routing_key: Optional[str] = None) -> dict:
        mgr = self.teachers.managers[self._resolve_teacher_key(routing_key)]
        ids, lps = await mgr.compute_topk_logprobs(request_id, list(prompt_ids) + list(response_ids))
        # row t predicts token t+1: the response tokens are predicted by rows [len(prompt)-1, len(prompt)+len(resp)-1)
        lo = len(prompt_ids) - 1
        ids, lps = ids[lo : lo + len(response_ids)], lps[lo : lo + len(response_ids)]
        pi, pl = pad_teacher_outputs(ids, lps, self.response_length, self.pad_token_id)
        return {"teacher_ids": pi, "teacher_logprobs": pl}
