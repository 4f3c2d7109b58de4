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


# ---------------------------------------------------------------------------------------------------------------------
# tools declared by decorating plain functions in a user's Python file (``rollout.multi_turn.function_tool_path``)
FUNCTION_TOOL_REGISTRY: dict[str, FunctionTool] = {}
_LOADED_FUNCTION_TOOL_PATHS: dict[str, list] = {}


def function_tool(fn: Optional[Callable] = None, *, name: Optional[str] = None, description: Optional[str] = None):
    """``@function_tool`` or ``@function_tool(name=..., description=...)``: the function becomes a tool whose schema is read
    from its signature and docstring; it stays callable as before. Variadic parameters cannot be put in a schema and are
    refused; so is a second tool of the same name. Parity target: ``verl/tools/function_tool.py`` (decorator and
    ``load_function_tools_from_path`` :151-184)."""

    def wrap(f: Callable):
        tool_name = name or f.__name__
        variadic = [n for n, p in inspect.signature(f).parameters.items()
                    if p.kind in (inspect.Parameter.VAR_POSITIONAL, inspect.Parameter.VAR_KEYWORD)]
        if variadic:
            raise ValueError(f"@function_tool '{tool_name}' ({f.__module__}.{f.__qualname__}) declares variadic parameter(s) "
                             f"{variadic}, which can't be expressed in an OpenAI tool schema. Replace them with explicit named "
                             f"parameters.")
        if tool_name in FUNCTION_TOOL_REGISTRY and FUNCTION_TOOL_REGISTRY[tool_name].fn is not f:
            raise ValueError(f"a function tool named '{tool_name}' is already registered")
        FUNCTION_TOOL_REGISTRY[tool_name] = FunctionTool(f, name=tool_name, description=description)
        return f

    return wrap(fn) if fn is not None else wrap


def get_function_tool(name: str) -> FunctionTool:
    return FUNCTION_TOOL_REGISTRY[name]


def load_function_tools_from_path(path: str) -> list:
    """Run the Python file at ``path`` once and return the tools its ``@function_tool`` decorators registered."""
    import importlib.util
    import logging
    import os
    import sys

    abs_path = os.path.abspath(path)
    if not os.path.isfile(abs_path):
        raise FileNotFoundError(f"function_tool_path does not exist: {path}")
    if abs_path in _LOADED_FUNCTION_TOOL_PATHS:
        return _LOADED_FUNCTION_TOOL_PATHS[abs_path]
    before = set(FUNCTION_TOOL_REGISTRY)
    # a module name derived from the path: the file can be found in sys.modules by what it imports, two files never clash
    mod_name = "_verl_function_tools_" + abs_path.replace(os.sep, "_").replace(".", "_")
    spec = importlib.util.spec_from_file_location(mod_name, abs_path)
    if spec is None or spec.loader is None:
        raise ImportError(f"Cannot create import spec for function_tool_path: {path}")
    module = importlib.util.module_from_spec(spec)
    sys.modules[mod_name] = module
    spec.loader.exec_module(module)
    new = sorted(set(FUNCTION_TOOL_REGISTRY) - before)
    if not new:
        logging.getLogger(__name__).warning("function_tool_path '%s' loaded but no @function_tool decorators found; did you "
                                            "forget to apply the decorator?", path)
    tools = [FUNCTION_TOOL_REGISTRY[n] for n in new]
    _LOADED_FUNCTION_TOOL_PATHS[abs_path] = tools
    return tools
