"""Cache-free sampling loop: every new token re-runs the whole prefix through the trainer's own model.

Slow by construction; it is the numerics oracle for the paged engine (no KV cache, no paging, no graph) and the
fallback when no rollout engine is configured. Parity target: ``verl/workers/rollout/naive/naive_rollout.py:36-120``
(left-padded prompts, one token per step, attention mask extended by ``prev != eos``, returns ``old_log_probs``).
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch

from ....models.decoder import DecoderModel, PackedBatch
from ....protocol import DataProto
from ....utils.tensordict_lite import TensorDict
from ..base import BaseRollout

__all__ = ["NaiveRollout", "last_token_logits", "filter_logits"]


def last_token_logits(model: DecoderModel, input_ids: torch.Tensor, attention_mask: torch.Tensor,
                      position_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 logits [b, V] at the last column of a left-padded batch (padding removed before the forward)."""
    mask = attention_mask.bool()
    lens = mask.sum(-1)
    ids = input_ids[mask]
    pos = (torch.cumsum(mask.to(torch.int32), -1) - 1)[mask] if position_ids is None else position_ids[mask]
    cu = torch.zeros(lens.numel() + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens.cpu().to(torch.int32), 0)
    batch = PackedBatch(input_ids=ids.contiguous(), positions=pos.to(torch.int32).contiguous(),
                        cu_seqlens=cu.to(input_ids.device), max_seqlen=int(lens.max()), cu_seqlens_cpu=cu)
    logits = model.forward_logits(batch)  # [T, V]
    last = (cu[1:].to(torch.int64) - 1).to(logits.device)
    return logits[last].float()


def filter_logits(logits: torch.Tensor, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """Mask everything outside the top-k set and outside the smallest set whose mass reaches top-p."""
    if top_k and top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.size(-1)), dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        srt, order = torch.sort(logits, dim=-1, descending=True)
        cum = torch.softmax(srt, -1).cumsum(-1)
        drop = cum - torch.softmax(srt, -1) >= top_p  # keep the token that crosses the threshold
        srt = srt.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, order, srt)
    return logits


class NaiveRollout(BaseRollout):
    def __init__(self, module: DecoderModel, config, model_config=None, device_mesh=None):
        super().__init__(config, model_config, device_mesh)
        self.module = module

    async def resume(self, tags: list[str]):
        return None

    async def release(self):
        return None

    async def update_weights(self, weights: Iterable, **kwargs):
        # shares the trainer's flat buffer: nothing to copy
        for _ in weights:
            pass

    def _cfg(self, key, default=None):
        c = self.config
        return c.get(key, default) if hasattr(c, "get") else getattr(c, key, default)

    @torch.no_grad()
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        idx = prompts.batch["input_ids"]
        attention_mask = prompts.batch["attention_mask"]
        position_ids = prompts.batch["position_ids"] if "position_ids" in prompts.batch.keys() else (
            torch.cumsum(attention_mask, -1) - 1).clamp_min(0)
        eos = prompts.meta_info.get("eos_token_id", [])
        eos = [eos] if isinstance(eos, int) else list(eos or [])
        b, P = idx.shape
        R = int(self._cfg("response_length"))
        temperature = float(prompts.meta_info.get("temperature", self._cfg("temperature", 1.0)))
        do_sample = bool(prompts.meta_info.get("do_sample", self._cfg("do_sample", True)))
        top_k = self._cfg("top_k", None)
        gen = None
        if prompts.meta_info.get("seed") is not None:
            gen = torch.Generator(device=idx.device).manual_seed(int(prompts.meta_info["seed"]))
        alive = torch.ones(b, 1, dtype=attention_mask.dtype, device=idx.device)
        step_logits = []
        for _ in range(R):
            logits = last_token_logits(self.module, idx, attention_mask, position_ids) / max(temperature, 1e-8)
            logits = filter_logits(logits, int(top_k) if top_k and top_k > 0 else 0)
            probs = torch.softmax(logits, -1)
            nxt = torch.multinomial(probs, 1, generator=gen) if do_sample else probs.argmax(-1, keepdim=True)
            attention_mask = torch.cat([attention_mask, alive], -1)
            for e in eos:
                alive = (alive.bool() & (nxt != e)).to(attention_mask.dtype)
            position_ids = torch.cat([position_ids, position_ids[:, -1:] + 1], -1)
            idx = torch.cat([idx, nxt], 1)
            step_logits.append(logits)
        logits = torch.stack(step_logits, 1)
        response = idx[:, P:]
        logp = torch.log_softmax(logits, -1).gather(-1, response.unsqueeze(-1)).squeeze(-1)
        batch = TensorDict({"prompts": idx[:, :P], "input_ids": idx, "responses": response, "sequences": idx,
                            "old_log_probs": logp, "rollout_log_probs": logp, "attention_mask": attention_mask,
                            "position_ids": position_ids, "response_mask": attention_mask[:, P:]}, batch_size=b)
        return DataProto(batch=batch, meta_info=dict(prompts.meta_info))
