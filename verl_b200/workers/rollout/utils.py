"""Small helpers shared by the rollout back-ends.

Parity target: ``verl/workers/rollout/utils.py`` (``get_max_position_embeddings`` :31, ``ensure_async_iterator`` :83,
``qwen2_5_vl_dedup_image_tokens`` :93, ``get_vision_placeholder_token_ids`` :117).
"""

from __future__ import annotations

from typing import Any, Optional

import numpy as np

__all__ = ["get_max_position_embeddings", "ensure_async_iterator", "dedup_vision_placeholder_runs", "qwen2_5_vl_dedup_image_tokens",
           "get_vision_placeholder_token_ids"]


def get_max_position_embeddings(hf_config: Any) -> int:
    """Context length of a model config; vision-language configs keep it on their ``text_config``."""
    for cfg in (hf_config, getattr(hf_config, "text_config", None)):
        n = getattr(cfg, "max_position_embeddings", None) if cfg is not None else None
        if n is not None:
            return int(n)
    raise ValueError("max_position_embeddings not found in HFModelConfig!")


async def ensure_async_iterator(iterable):
    """Iterate a plain or an asynchronous iterable with ``async for``."""
    if hasattr(iterable, "__aiter__"):
        async for item in iterable:
            yield item
    else:
        for item in iterable:
            yield item


def _placeholder_id(processor: Any, modality: str) -> Optional[int]:
    if processor is None:
        return None
    tid = getattr(processor, f"{modality}_token_id", None)
    if tid is None:
        token = getattr(processor, f"{modality}_token", None)
        tok = getattr(processor, "tokenizer", None)
        if token is not None and tok is not None and hasattr(tok, "convert_tokens_to_ids"):
            tid = tok.convert_tokens_to_ids(token)
    return None if tid is None else int(tid)


def get_vision_placeholder_token_ids(processor: Any) -> list[int]:
    """Image / video placeholder ids, which sampling must never produce: the k-th run of placeholders stands for the k-th
    image or video that was fed in, so a placeholder the model invents has nothing behind it and breaks the position and
    embedding bookkeeping of every consumer. Empty for text-only models (sampling is left alone)."""
    return [t for t in (_placeholder_id(processor, m) for m in ("image", "video")) if t is not None]


def dedup_vision_placeholder_runs(prompt_ids: list[int], placeholder_ids: list[int]) -> list[int]:
    """Collapse every run of consecutive placeholder tokens to its first token."""
    if not placeholder_ids or not prompt_ids:
        return list(prompt_ids)
    ids = np.asarray(prompt_ids)
    is_ph = np.isin(ids, np.asarray(placeholder_ids))
    keep = np.ones(len(ids), dtype=bool)
    keep[1:] &= ~(is_ph[1:] & is_ph[:-1])
    return ids[keep].tolist()


def qwen2_5_vl_dedup_image_tokens(prompt_ids: list[int], processor: Any) -> list[int]:
    """A prompt rendered by a Qwen2-VL style processor repeats ``<|image_pad|>`` once per patch; a server that expands the
    placeholder itself from the image data wants it once per image: ``<|vision_start|><|image_pad|>...<|image_pad|>
    <|vision_end|>`` becomes ``<|vision_start|><|image_pad|><|vision_end|>``. Other processors: unchanged."""
    ip = getattr(processor, "image_processor", None)
    if ip is None or "Qwen2VLImageProcessor" not in type(ip).__name__:
        return prompt_ids
    return dedup_vision_placeholder_runs(prompt_ids, get_vision_placeholder_token_ids(processor))
