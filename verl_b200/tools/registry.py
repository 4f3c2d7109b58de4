"""Tool loading from a YAML/JSON list. Parity target: ``verl/tools/utils/tool_registry.py`` (101 lines)."""

from __future__ import annotations

import importlib
import json
from typing import Optional

import yaml

from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema

__all__ = ["initialize_tools_from_config", "get_tool_class"]


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
