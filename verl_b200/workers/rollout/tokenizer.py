"""Minimal tokenizer interface the rollout / reward code relies on, so that engines can be driven by something other than a
HuggingFace tokenizer (a sentencepiece model, a test stub).

Parity target: ``verl/workers/rollout/tokenizer.py`` (``HybridEngineBaseTokenizer`` :26).
"""

from __future__ import annotations

from abc import ABC, abstractmethod

__all__ = ["HybridEngineBaseTokenizer"]


class HybridEngineBaseTokenizer(ABC):
    @property
    @abstractmethod
    def vocab_size(self) -> int: ...

    @property
    @abstractmethod
    def pad_token_id(self) -> int: ...

    @property
    @abstractmethod
    def eos_token_id(self) -> int: ...

    @property
    def all_special_ids(self) -> list[int]:
        return [i for i in {self.pad_token_id, self.eos_token_id} if i is not None]

    @property
    def all_special_tokens(self) -> list[str]:
        return self.convert_ids_to_tokens(self.all_special_ids)

    @abstractmethod
    def encode(self, text: str) -> list[int]: ...

    @abstractmethod
    def decode(self, token_ids, skip_special_tokens: bool = False, clean_up_tokenization_spaces=None, **kwargs) -> str: ...

    @abstractmethod
    def convert_ids_to_tokens(self, ids, skip_special_tokens: bool = False): ...

    def get_added_vocab(self) -> dict[str, int]:
        return {}

    def convert_tokens_to_string(self, tokens: list[str]) -> str:
        return "".join(tokens)

    @property
    def is_fast(self) -> bool:
        return False
