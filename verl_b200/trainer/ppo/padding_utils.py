"""No-op padding samples that make a sampled batch divisible by the data-parallel / mini-batch layout.

A padding sample is a one-token prompt plus a one-token response of EOS with ``response_mask`` zero, zero scores and zero
rollout log-probs: it flows through every pass but contributes to no loss, entropy or KL term; its tag carries
``is_padding`` so that metrics can skip it.

Parity target: ``verl/trainer/ppo/padding_utils.py`` (``build_padding_position_ids`` :43, ``build_padding_routed_experts`` :57,
``construct_minimal_padding_template`` :70, ``upsample_batch_to_divisible_size`` :127).
"""

from __future__ import annotations

import copy
import uuid
from typing import Any, Optional

import torch

from ...utils import torch_functional as VF
from ...utils.transfer_queue import KVBatchMeta, TransferQueue

__all__ = ["build_padding_position_ids", "build_padding_routed_experts", "construct_minimal_padding_template",
           "upsample_batch_to_divisible_size"]


def build_padding_position_ids(source_position_ids: Any, attention_mask: torch.Tensor) -> torch.Tensor:
    """Position ids of the padding sample with the rank / leading dims of the source sample's (e.g. 3-row mrope ids)."""
    pos = VF.compute_position_id_with_mask(attention_mask.unsqueeze(0)).squeeze(0)
    if not isinstance(source_position_ids, torch.Tensor):
        return pos
    pos = pos.to(device=source_position_ids.device, dtype=source_position_ids.dtype)
    if source_position_ids.dim() <= 1:
        return pos
    shape = (1,) * (source_position_ids.dim() - 1) + (pos.size(-1),)
    return pos.reshape(shape).expand(*source_position_ids.shape[:-1], -1).clone()


def build_padding_routed_experts(source_routed_experts: Any, seq_len: int) -> Optional[torch.Tensor]:
    if not isinstance(source_routed_experts, torch.Tensor):
        return None
    if source_routed_experts.dim() == 0:
        return torch.zeros_like(source_routed_experts)
    return torch.zeros((seq_len, *source_routed_experts.shape[1:]), dtype=source_routed_experts.dtype, device=source_routed_experts.device)


def construct_minimal_padding_template(source: dict, source_tag: dict, eos_token_id: int) -> tuple[dict, dict]:
    sample = {k: (v.clone() if isinstance(v, torch.Tensor) else copy.deepcopy(v)) for k, v in source.items()}
    tag = copy.deepcopy(source_tag)
    prompts = torch.full((1,), int(eos_token_id), dtype=torch.int64)
    input_ids = prompts.repeat(2)
    am = torch.ones_like(input_ids)
    rmask = torch.zeros_like(prompts)
    sample.update(prompts=prompts, responses=prompts.clone(), input_ids=input_ids, attention_mask=am,
                  position_ids=build_padding_position_ids(sample.get("position_ids"), am), num_turns=0, response_mask=rmask, loss_mask=rmask,
                  rm_scores=torch.zeros(1, dtype=torch.float32), rollout_log_probs=torch.zeros(1, dtype=torch.float32))
    if "multi_modal_inputs" in sample:
        sample["multi_modal_inputs"] = {}
    routed = build_padding_routed_experts(source.get("routed_experts"), 2)
    if routed is not None:
        sample["routed_experts"] = routed
    else:
        sample.pop("routed_experts", None)
    tag.update(is_padding=True, prompt_len=1, response_len=1, seq_len=2)
    return sample, tag


def upsample_batch_to_divisible_size(batch: KVBatchMeta, batch_multiple: int, eos_token_id: int, queue: TransferQueue) -> KVBatchMeta:
    """Append padding samples (stored in ``queue`` like real ones) until ``len(batch) % batch_multiple == 0``."""
    rem = len(batch) % batch_multiple
    if rem == 0 or len(batch) == 0:
        return batch
    src = queue.get([batch.keys[0]], None, batch.partition_id)[0]
    tmpl, tag = construct_minimal_padding_template(src, batch.tags[0] if batch.tags else {}, eos_token_id)
    uid = f"pad{uuid.uuid4().hex}"
    keys, tags = list(batch.keys), list(batch.tags)
    for i in range(batch_multiple - rem):
        key = f"{uid}_{i}_0"
        sample = {k: (v.clone() if isinstance(v, torch.Tensor) else copy.deepcopy(v)) for k, v in tmpl.items()}
        sample["uid"] = uid
        queue.put(key, sample, dict(tag, kind="traj", uid=uid), batch.partition_id)
        keys.append(key)
        tags.append(dict(tag))
    return KVBatchMeta(keys, batch.partition_id, batch.fields, tags)
