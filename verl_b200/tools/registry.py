"""Tool loading from a YAML/JSON list. Parity target: ``verl/tools/utils/tool_registry.py`` (101 lines)."""

from __future__ import annotations

import importlib
import json
from typing import Optional

import yaml

from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema

__all__ = ["initialize_tools_from_config", "get_tool_class", "load_all_tools"]


def get_tool_class(cls_name: str):
    mod, _, name = cls_name.rpartition(".")
    mod = mod.replace("verl.", "verl_b200.", 1) if mod.startswith("verl.") else mod
    return getattr(importlib.import_module(mod), name)


def initialize_tools_from_config(tools_config_file: Optional[str]) -> list[BaseTool]:
    if not tools_config_file:
        return []
    with open(tools_config_file) as f:
        cfg = json.load(f) if tools_config_file.endswith(".json") else yaml.safe_load(f)
    tools = []
    for item in cfg.get("tools", []):
        cls = get_tool_class(item["class_name"])
        schema = OpenAIFunctionToolSchema.model_validate(item["tool_schema"]) if item.get("tool_schema") else None
        tools.append(cls(config=item.get("config", {}), tool_schema=schema))
    return tools


def load_all_tools(tool_config_path: Optional[str], function_tool_path: Optional[str]) -> list:
    """Tools declared in the YAML file plus tools declared by ``@function_tool`` in a Python file; a name may come from
    one of the two only. Parity target: ``verl/tools/tool_registry.py:83-101``."""
    from .function_tool import load_function_tools_from_path

    native = initialize_tools_from_config(tool_config_path) if tool_config_path else []
    functions = load_function_tools_from_path(function_tool_path) if function_tool_path else []
    clash = sorted({t.name for t in native} & {t.name for t in functions})
    if clash:
        raise ValueError(f"Function tool name(s) {clash} collide with tools already declared in '{tool_config_path}'. Each tool "
                         f"name must be unique across `tool_config_path` and `function_tool_path`; rename one of them.")
    return native + functions
