"""Extraction of tool calls from generated text.

Parity target: ``verl/experimental/agent_loop/tool_parser.py`` (816 lines): a registry of model-family parsers
(hermes ``<tool_call>{json}</tool_call>``, gpt-oss channel format, Qwen3-coder XML, Llama-3 JSON).
"""

from __future__ import annotations

import json
import re
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Optional

__all__ = ["FunctionCall", "ToolParser", "HermesToolParser", "GptOssToolParser", "Qwen3XMLToolParser",
           "Llama3JsonToolParser"]


@dataclass
class FunctionCall:
    name: str
    arguments: str  # JSON string


class ToolParser(ABC):
    _registry: dict[str, type["ToolParser"]] = {}

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer

    @abstractmethod
    async def extract_tool_calls(self, responses_ids: list[int], text: Optional[str] = None) -> tuple[str, list[FunctionCall]]:
        """Returns (content with the tool-call markup removed, calls)."""

    def _text(self, ids, text):
        if text is not None:
            return text
        return self.tokenizer.decode(ids) if self.tokenizer is not None else ""

    @classmethod
    def get_tool_parser(cls, name: str, tokenizer=None) -> "ToolParser":
        if name not in cls._registry:
            raise ValueError(f"Unknown tool parser: {name} (known: {sorted(cls._registry)})")
        return cls._registry[name](tokenizer)

    @classmethod
    def register(cls, name: str):
        def deco(sub):
            cls._registry[name] = sub
            return sub

        return deco


@ToolParser.register("hermes")
class HermesToolParser(ToolParser):
    PAT = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)

    async def extract_tool_calls(self, responses_ids, text=None):
        text = self._text(responses_ids, text)
        if "<tool_call>" not in text:
            return text, []
        calls = []
        for m in self.PAT.findall(text):
            try:
                obj = json.loads(m)
                calls.append(FunctionCall(name=obj["name"], arguments=json.dumps(obj.get("arguments", {}), ensure_ascii=False)))
            except Exception:
                continue
        return self.PAT.sub("", text), calls


@ToolParser.register("gpt-oss")
class GptOssToolParser(ToolParser):
    """``<|start|>assistant<|channel|>commentary to=functions.NAME <|constrain|>json<|message|>{...}<|call|>``"""

    PAT = re.compile(r"to=functions\.([\w\-\.]+).*?<\|message\|>(.*?)(?:<\|call\|>|$)", re.DOTALL)
    COT = re.compile(r"<\|channel\|>analysis<\|message\|>.*?<\|end\|>", re.DOTALL)

    async def extract_tool_calls(self, responses_ids, text=None):
        text = self.COT.sub("", self._text(responses_ids, text))
        calls = []
        for name, args in self.PAT.findall(text):
            try:
                json.loads(args)
                calls.append(FunctionCall(name=name, arguments=args.strip()))
            except Exception:
                continue
        return self.PAT.sub("", text), calls


@ToolParser.register("qwen3_xml")
class Qwen3XMLToolParser(ToolParser):
    """``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``"""

    CALL = re.compile(r"<tool_call>\s*<function=([^>]+)>(.*?)</function>\s*</tool_call>", re.DOTALL)
    PARAM = re.compile(r"<parameter=([^>]+)>(.*?)</parameter>", re.DOTALL)

    async def extract_tool_calls(self, responses_ids, text=None):
        text = self._text(responses_ids, text)
        calls = []
        for name, body in self.CALL.findall(text):
            args = {}
            for k, v in self.PARAM.findall(body):
                v = v.strip()
                try:
                    args[k.strip()] = json.loads(v)
                except Exception:
                    args[k.strip()] = v
            calls.append(FunctionCall(name=name.strip(), arguments=json.dumps(args, ensure_ascii=False)))
        return self.CALL.sub("", text), calls


@ToolParser.register("llama3_json")
class Llama3JsonToolParser(ToolParser):
    """A bare JSON object ``{"name": ..., "parameters": {...}}`` (optionally after ``<|python_tag|>``)."""

    async def extract_tool_calls(self, responses_ids, text=None):
        text = self._text(responses_ids, text)
        body = text.split("<|python_tag|>")[-1].strip()
        calls = []
        for chunk in body.split(";"):
            chunk = chunk.strip()
            if not chunk.startswith("{"):
                continue
            try:
                obj = json.loads(chunk)
                calls.append(FunctionCall(name=obj["name"], arguments=json.dumps(obj.get("parameters", obj.get("arguments", {})))))
            except Exception:
                continue
        return ("" if calls else text), calls
