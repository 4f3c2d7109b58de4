"""Wrap a plain python function as a tool; the schema is derived from the signature and docstring.

Parity target: ``verl/tools/function_tool.py`` (258 lines)."""

from __future__ import annotations

import asyncio
import inspect
import json
from typing import Any, Callable, Optional, get_type_hints

from .base_tool import BaseTool
from .schemas import (OpenAIFunctionParametersSchema, OpenAIFunctionPropertySchema, OpenAIFunctionSchema,
                      OpenAIFunctionToolSchema, ToolResponse)

__all__ = ["FunctionTool", "function_to_schema"]

_JSON_TYPES = {int: "integer", float: "number", str: "string", bool: "boolean", list: "array", dict: "object"}


def function_to_schema(fn: Callable, name: Optional[str] = None, description: Optional[str] = None) -> OpenAIFunctionToolSchema:
    sig = inspect.signature(fn)
    hints = get_type_hints(fn) if callable(fn) else {}
    doc = inspect.getdoc(fn) or ""
    arg_docs = {}
    for line in doc.splitlines():
        line = line.strip()
        if ":" in line and line.split(":")[0].split("(")[0].strip() in sig.parameters:
            k, v = line.split(":", 1)
            arg_docs[k.split("(")[0].strip()] = v.strip()
    props, required = {}, []
    for pname, p in sig.parameters.items():
        if pname in ("self", "kwargs", "args") or p.kind in (p.VAR_KEYWORD, p.VAR_POSITIONAL):
            continue
        t = hints.get(pname, str)
        props[pname] = OpenAIFunctionPropertySchema(type=_JSON_TYPES.get(getattr(t, "__origin__", t), "string"),
                                                    description=arg_docs.get(pname))
        if p.default is inspect._empty:
            required.append(pname)
    return OpenAIFunctionToolSchema(function=OpenAIFunctionSchema(
        name=name or fn.__name__, description=description or (doc.split("\n\n")[0] if doc else ""),
        parameters=OpenAIFunctionParametersSchema(properties=props, required=required)))


class FunctionTool(BaseTool):
    def __init__(self, fn: Callable, config: Optional[dict] = None, tool_schema: Optional[OpenAIFunctionToolSchema] = None,
                 name: Optional[str] = None, description: Optional[str] = None):
        self.fn = fn
        super().__init__(config or {}, tool_schema or function_to_schema(fn, name, description))

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs) -> tuple[ToolResponse, float, dict]:
        try:
            res = self.fn(**parameters)
            if inspect.isawaitable(res):
                res = await res
        except Exception as e:  # tool errors are observations for the model, not crashes of the rollout
            return ToolResponse(text=f"Error when executing tool: {e}"), 0.0, {"tool_error": 1}
        if isinstance(res, ToolResponse):
            return res, 0.0, {}
        text = res if isinstance(res, str) else json.dumps(res, ensure_ascii=False, default=str)
        return ToolResponse(text=text), 0.0, {}
