"""Tokenizer / processor loading. Parity target: ``verl/utils/tokenizer/tokenizer.py`` (252 lines)."""

from __future__ import annotations

import warnings

__all__ = ["hf_tokenizer", "hf_processor", "set_pad_token_id"]


def set_pad_token_id(tokenizer) -> None:
    if tokenizer.pad_token_id is None:
        tokenizer.pad_token_id = tokenizer.eos_token_id
        warnings.warn(f"tokenizer.pad_token_id is None. Now set to {tokenizer.eos_token_id}", stacklevel=1)
    if tokenizer.pad_token is None:
        tokenizer.pad_token = tokenizer.eos_token


def hf_tokenizer(name_or_path, correct_pad_token: bool = True, correct_gemma2: bool = True, **kwargs):
    from transformers import AutoTokenizer

    if correct_gemma2 and isinstance(name_or_path, str) and "gemma-2-2b-it" in name_or_path:
        kwargs["eos_token"] = "<end_of_turn>"
        kwargs["eos_token_id"] = 107
    tok = AutoTokenizer.from_pretrained(name_or_path, **kwargs)
    if correct_pad_token:
        set_pad_token_id(tok)
    return tok


def hf_processor(name_or_path, **kwargs):
    from transformers import AutoProcessor

    try:
        proc = AutoProcessor.from_pretrained(name_or_path, **kwargs)
    except Exception as e:
        warnings.warn(f"Failed to create processor: {e}. This may affect multimodal processing", stacklevel=1)
        return None
    if proc is not None and "Processor" not in proc.__class__.__name__:
        return None
    return proc
